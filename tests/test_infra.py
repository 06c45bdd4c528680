"""Arena / scratch registry / logger."""
import pytest
import torch

from volta_engine_b200.runtime.arena import Arena, ArenaError, ScratchRegistry
from volta_engine_b200.utils import log


def test_arena_bump_alignment_freeze_and_release():
    a = Arena(1 << 16, "cpu")
    x = a.alloc((3, 5), torch.float32, "w/a")
    y = a.alloc(100, torch.uint8, "w/b")
    assert x.shape == (3, 5) and x.dtype == torch.float32
    assert x.data_ptr() % 256 == 0 and y.data_ptr() % 256 == 0 and y.data_ptr() - x.data_ptr() == 256
    x.fill_(1.0); y.fill_(7)
    assert float(x.sum()) == 15.0                     # no overlap
    mark = a.mark()
    a.alloc(1000, name="tmp/c")
    a.release_to(mark)
    z = a.alloc(8, name="w/d")
    assert z.data_ptr() - y.data_ptr() == 256
    rep = a.report()
    assert rep["by_name"]["w"] == 60 + 100 + 8 and rep["high_water"] >= rep["used"]
    with pytest.raises(ArenaError):
        a.alloc(1 << 20, name="too-big")
    a.freeze()
    with pytest.raises(ArenaError):
        a.alloc(8, name="late")


def test_scratch_registry_returns_stable_memory():
    a = Arena(1 << 16, "cpu")
    s = ScratchRegistry(a)
    p = s.get("splitk", 1024)
    assert s.get("splitk", 512).data_ptr() == p.data_ptr()
    t = s.typed("recon", (4, 8), torch.bfloat16)
    assert t.shape == (4, 8) and s.typed("recon", (2, 8), torch.bfloat16).data_ptr() == t.data_ptr()
    grown = s.get("splitk", 4096)
    assert grown.numel() >= 4096
    a.freeze()
    assert s.get("splitk", 100).data_ptr() == grown.data_ptr()
    with pytest.raises(ArenaError):
        s.get("splitk", 1 << 15)
    assert s.total_bytes() >= 4096 + 64


def test_logger_levels(capsys):
    log.set_level("warn")
    log.info("hidden %d", 1)
    log.warn("shown %s", "w")
    log.error("bad")
    out = capsys.readouterr()
    assert out.out == "" and "WARN  shown w" in out.err and "ERROR bad" in out.err
    log.set_level("debug")
    log.debug("dbg %.1f", 2.5)
    assert "DEBUG dbg 2.5" in capsys.readouterr().out
    log.set_level("info")
    with pytest.raises(ValueError):
        log.set_level("loud")


def test_capability_table_covers_every_exported_kernel():
    from volta_engine_b200.utils import capabilities as C
    assert C.missing() == []
    assert [k for k in C.TABLE if k not in C.exported()] == []
    md = C.markdown()
    assert "| Attention | `ve_attention` | portable |" in md and "| Collectives | `ve_ll_allreduce` | device |" in md


def test_every_programmatically_launched_kernel_waits_for_its_predecessor():
    """A kernel launched with programmatic stream serialization starts before the kernel in front has finished; one that
    never executes the dependency wait reads half-written inputs once launches overlap (CUDA-graph replay) while eager
    runs look fine. Every kernel named at a launch_pdl call site must contain grid_dep_wait()."""
    import glob
    import os
    import re
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "volta_engine_b200", "csrc", "cuda")
    seen = 0
    for path in glob.glob(os.path.join(root, "*.cu")):
        src = open(path).read()
        for name in set(re.findall(r"launch_pdl\(\s*([A-Za-z_0-9]+)", src)):
            m = re.search(r"__global__[^;{]*?\b" + name + r"\s*\(", src)
            assert m, f"{name}: definition not found in {path}"
            i = src.index("{", m.end())
            depth, j = 0, i
            while True:
                depth += src[j] == "{"
                depth -= src[j] == "}"
                if depth == 0:
                    break
                j += 1
            assert "grid_dep_wait" in src[i:j], f"{os.path.basename(path)}: {name} is launched programmatically but never waits"
            seen += 1
    assert seen >= 20
