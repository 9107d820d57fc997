"""The NVTX range helper (counterpart of kiln's kiln-nvtx crate, kiln-nvtx/src/lib.rs:26-84): off by default, and when
switched on it pushes and pops exactly once around the wrapped call, also when the call raises."""
import pytest

from kiln_b200 import nvtx


def test_ranges_are_off_by_default_and_balanced_when_on():
    log = []
    with nvtx.range("kiln/marlin/gemm"):
        pass
    assert log == []
    nvtx.enable(True, push=lambda name: log.append(("push", name)), pop=lambda: log.append(("pop",)))
    try:
        with nvtx.range("kiln/mlp/down"):
            log.append(("body",))
        with pytest.raises(ValueError):
            with nvtx.range("kiln/proj/grouped"):
                raise ValueError("boom")
    finally:
        nvtx.enable(False)
    assert log == [("push", "kiln/mlp/down"), ("body",), ("pop",), ("push", "kiln/proj/grouped"), ("pop",)]
    with nvtx.range("kiln/marlin/gemm"):
        pass
    assert len(log) == 5
