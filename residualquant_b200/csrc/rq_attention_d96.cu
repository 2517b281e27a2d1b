// Packed paged decode attention, head_dim 96 variants.
#define RQ_ATTENTION_HEAD_DIM 96
#include "rq_attention_impl.cuh"
