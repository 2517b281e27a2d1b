"""Host-side pieces of bench.py that need no GPU: the algorithmic-byte formulas behind `roofline.achieved`, the page
widths they rest on, and the command-line defaults the measurement contract fixes."""

import importlib.util
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    module = importlib.util.module_from_spec(spec)
    sys.modules["bench_under_test"] = module   # dataclasses look their module up by name
    spec.loader.exec_module(module)
    return module


def test_record_sizes_and_page_widths():
    b = _bench()
    # Bytes = D*bits/8 + 2*D/group + 2 (csrc/common/cache.cuh:14-17 of the reference)
    assert (b.record_bytes(4, 32, 128), b.record_bytes(2, 32, 128), b.record_bytes(2, 16, 128)) == (74, 42, 50)
    assert (b.record_bytes(4, 32, 96), b.record_bytes(2, 32, 96), b.record_bytes(2, 16, 96)) == (56, 32, 38)
    assert b.Shape(1, 1, 1).width == 200 and b.Shape(1, 1, 1, group=16).width == 224
    assert b.Shape(1, 1, 1, heads=55, head_dim=96).width == 152


def test_algorithmic_bytes_of_the_headline_point():
    b = _bench()
    shape = b.Shape(batch=64, context=8192, layers=24)
    history = 64 * 8191
    # residual loop: 228 bytes per cached token and head (K and V: anchor without its alpha column + one INT2 record)
    assert b.attention_bytes(history, 64, shape, False) == history * 16 * 228 + 64 * 16 * 128 * 8 == 1913417728
    assert b.attention_bytes(history, 64, shape, True) == history * 16 * 144 + 64 * 16 * 128 * 8
    # a write reads four loops of bf16 K and V and writes one page row per token, head and plane
    assert b.quantize_bytes(16384, shape) == 2 * 4 * 16384 * 16 * 128 * 2 + 2 * 16384 * 16 * 200
    d96 = b.Shape(batch=16, context=4096, layers=1, heads=55, head_dim=96)
    assert b.attention_bytes(16 * 4095, 16, d96, False) == 16 * 4095 * 55 * 172 + 16 * 55 * 96 * 8


def test_command_line_defaults(monkeypatch):
    b = _bench()
    monkeypatch.setattr(sys, "argv", ["bench.py"])
    args = b.parse_args()
    assert (args.gpus, args.impl, args.batch, args.context, args.layers) == (1, "b200", 64, 8192, 24)
    assert args.warmup >= 3 and 1 <= args.steps <= 64
    assert (b.METRIC, b.UNIT) == ("decode_tokens_per_s", "tokens/s")
