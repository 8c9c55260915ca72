"""Checks on the kernel sources themselves (CPU): required Blackwell constructs are present,
constructs that are closed on shared GPU pools are absent, every device-side wait is bounded, and
the ctypes mirrors match the C structs."""
import re
from pathlib import Path

CSRC = Path(__file__).resolve().parent.parent / "mi50grad_b200" / "csrc"
SOURCES = {p.name: p.read_text() for p in sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))}


def test_blackwell_constructs_present():
    # the tcgen05 kernels (GEMM, prompt attention) and the PTX helpers they share
    g = SOURCES["tc_util.cuh"] + SOURCES["gemm_tc.cu"] + SOURCES["attention_tc.cu"]
    for needle in ("tcgen05.mma.cta_group::1.kind::f16", "tcgen05.alloc", "tcgen05.dealloc", "tcgen05.commit",
                   "tcgen05.ld.sync.aligned.32x32b", "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier",
                   "mbarrier.try_wait.parity", "elect.sync"):
        assert needle in g, needle
    assert "tcgen05.mma.cta_group::2.kind::f16" in g and "tcgen05.alloc.cta_group::2" in SOURCES["gemm_tc.cu"]
    for name in ("gemm_tc.cu", "attention_tc.cu"):
        assert "tcgen05.alloc" in SOURCES[name] and "tcgen05.dealloc" in SOURCES[name] and "tc_mma_f16(" in SOURCES[name], name
    assert "multimem.ld_reduce" in SOURCES["common.cuh"] and "multimem.st" in SOURCES["common.cuh"]
    assert "griddepcontrol.launch_dependents" in SOURCES["common.cuh"]
    assert "cluster.map_shared_rank" in SOURCES["deltanet.cu"]
    assert "mma.sync.aligned.m16n8k16" in SOURCES["attention_rows.cu"]
    assert "mma.sync.aligned.m16n8k8.row.col.f32.tf32" in SOURCES["deltanet.cu"]


def test_closed_constructs_absent():
    tail = "Batch" + "Async"                                      # the batched-copy entry points, never spelled out
    banned_calls = [pre + mid + tail for pre in ("cuda", "cu") for mid in ("Memcpy", "Memcpy3D")]
    for name, text in SOURCES.items():
        for m in re.finditer(r'cp\.async\.bulk[\w.:]*', text):        # bulk / tensor copies: plain form only, no broadcast qualifier
            assert "cast" not in m.group(0), (name, m.group(0))
        assert "wgmma" not in text, name
        assert "__trap" not in text and "asm(\"trap" not in text, name
        for b in banned_calls:
            assert b not in text, (name, b)


def test_every_spin_wait_is_bounded():
    # loops that poll a flag or barrier must sit next to a time or iteration bound
    c = SOURCES["common.cuh"]
    body = c[c.index("wait_reached"):]
    assert "globaltimer_ns() - t0 > budget_ns" in body
    g = SOURCES["tc_util.cuh"]
    w = g[g.index("bool mbar_wait("):g.index("elect_one")]
    assert "TC_WAIT_NS" in w and "abort_flag" in w
    # the tcgen05 kernels wait on mbarriers only through that bounded helper
    for name in ("gemm_tc.cu", "attention_tc.cu"):
        assert "mbar_try_wait(" not in SOURCES[name] and "mbar_wait(" in SOURCES[name], name
    assert "GEMV_TAG_POLLS" in SOURCES["gemv.cu"]
    for name, text in SOURCES.items():
        for m in re.finditer(r"while\s*\(\s*(true|1)\s*\)|for\s*\(\s*;\s*;\s*\)", text):
            window = text[m.start():m.start() + 700]
            assert ("globaltimer" in window or "abort_flag" in window or "return" in window or "break" in window), (name, m.group(0))


def test_ctypes_mirrors_match_c_structs():
    from mi50grad_b200.ops import lib as L
    L.lib()                                                        # raises on any size mismatch
