"""The C-ABI library loads without a GPU and exports every function include/rq_b200.h declares (CPU)."""

import ctypes
import os
import re

import pytest

from residualquant_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "rq_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rq_[a-z_0-9]+)\s*\(", text)))


def test_header_and_binding_agree(built_library):
    declared = _declared_functions()
    assert declared, "no declarations found"
    assert sorted(_lib.EXPORTS) == declared
    lib = ctypes.CDLL(built_library)
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/rq_b200.h but not exported"


def test_layout_functions(built_library):
    lib = _lib.load()
    spec = _lib.make_spec([[2, 32]] * 3 + [[4, 32]], "anchor", 3, 16, 128, 16)
    assert lib.rq_page_width(ctypes.byref(spec)) == 200
    assert [lib.rq_record_offset(ctypes.byref(spec), i) for i in range(5)] == [0, 42, 84, 126, 200]
    spec = _lib.make_spec([[2, 16]] * 3 + [[4, 32]], "anchor", 3, 16, 128, 32)
    assert lib.rq_page_width(ctypes.byref(spec)) == 224
    spec = _lib.make_spec([[2, 32]] * 3 + [[4, 32]], "anchor", 3, 55, 96, 16)
    assert lib.rq_page_width(ctypes.byref(spec)) == 152
    spec = _lib.make_spec([[4, 32]], "anchor", 0, 16, 128, 16)
    assert lib.rq_page_width(ctypes.byref(spec)) == 74


def test_bad_specs_return_errors_not_crashes(built_library):
    lib = _lib.load()
    spec = _lib.make_spec([[3, 32]], "anchor", 0, 16, 128, 16)
    assert lib.rq_page_width(ctypes.byref(spec)) == -2
    assert b"bits=3" in lib.rq_last_error()
    spec = _lib.make_spec([[2, 32], [2, 32]], "adjacent", 1, 16, 128, 16)
    assert lib.rq_page_width(ctypes.byref(spec)) == -1
    spec = _lib.make_spec([[2, 32]], "anchor", 0, 16, 64, 16)
    assert lib.rq_page_width(ctypes.byref(spec)) == -2
    with pytest.raises(RuntimeError):
        _lib.make_spec([[2, 32]], "sideways", 0, 16, 128, 16)
    assert lib.rq_quantize(None) == -1
    assert lib.rq_attention(None) == -1


def test_workspace_size_and_split_heuristic(built_library):
    lib = _lib.load()
    one = lib.rq_attention_workspace_bytes(64, 16, 128, 1)
    four = lib.rq_attention_workspace_bytes(64, 16, 128, 4)
    assert one == 256 + 65536 and four == one + 64 * 16 * 4 * 130 * 4
    # the counter region is shape-independent up to 16384 (row, head) pairs, then the next power of two
    assert lib.rq_attention_workspace_bytes(1, 1, 128, 1) == 256 + 65536
    assert lib.rq_attention_workspace_bytes(2048, 16, 128, 1) == 256 + 131072
    assert four % 256 == 0
    # num_splits 0: sized for the work capacity, which depends on rows, heads and the SM count only (148 without a GPU)
    capacity = lib.rq_attention_work_capacity(64, 16)
    assert capacity == 64 + ((4 * 148 + 15) // 16 + 1) // 2        # several waves of rows: half a wave of spare items
    assert lib.rq_attention_work_capacity(32, 16) == 32 + 37           # less than a wave of rows: one wave of spare items
    assert lib.rq_attention_work_capacity(40, 16) == 80                # 1.08 waves of rows: room for two partitions per row
    assert lib.rq_attention_work_capacity(1, 16) == 16                 # a single row: its sixteen partitions
    assert lib.rq_attention_workspace_bytes(64, 16, 128, 0) == one + (capacity * 16 * 130 * 4 + 255) // 256 * 256
    assert lib.rq_attention_work_capacity(1, 16) == 16 and lib.rq_attention_work_capacity(0, 16) == 0
    assert lib.rq_attention_workspace_bytes(64, 16, 128, -100000) == 0
    assert 1 <= lib.rq_attention_default_splits(1, 16, 512, 16) <= 64
    assert lib.rq_attention_default_splits(1, 16, 512, 16) >= lib.rq_attention_default_splits(64, 16, 512, 16)
    assert lib.rq_attention_default_splits(64, 16, 1, 16) == 1
    spec = _lib.make_spec([[2, 32]] * 3 + [[4, 32]], "anchor", 3, 16, 128, 16)
    # dense rotations are applied inside the quantizer: no scratch for any rotation kind
    assert lib.rq_quantize_workspace_bytes(ctypes.byref(spec), 100, 1, 1) == 0
    assert lib.rq_quantize_workspace_bytes(ctypes.byref(spec), 100, 2, 2) == 0


def test_regular_build_carries_no_phase_timestamps(built_library):
    """The phase timestamps of the attention kernels exist only in the separate timeline build (build.py --timeline)."""
    lib = _lib.load()
    assert not hasattr(lib, "rq_timeline_d128") and not hasattr(lib, "rq_timeline_d96")


def test_timeline_script_and_kernel_agree_on_the_slots():
    """The phase-timestamp slots are named twice: in the kernel's enum and in the script that reads them back."""
    import os
    import re

    from residualquant_b200 import timeline

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    source = open(os.path.join(root, "residualquant_b200", "csrc", "rq_attention_impl.cuh")).read()
    body = re.search(r"enum TimelineSlot \{(.*?)\};", source, re.S).group(1)
    names = [n.split("=")[0].strip() for n in body.replace("\n", " ").split(",") if n.strip()]
    assert names[-1] == "kTimelineSlots" and len(names) - 1 == len(timeline.SLOTS)
    assert int(re.search(r"kTimelineCtas = (\d+)", source).group(1)) == timeline.TIMELINE_CTAS
    used = {slot for _, start, stop in timeline.PHASES for slot in (start, stop)}
    assert used <= set(timeline.SLOTS)
