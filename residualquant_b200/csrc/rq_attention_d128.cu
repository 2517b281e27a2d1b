// Packed paged decode attention, head_dim 128 variants.
#define RQ_ATTENTION_HEAD_DIM 128
#include "rq_attention_impl.cuh"
