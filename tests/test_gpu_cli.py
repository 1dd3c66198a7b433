"""The native benchmark / parity command line (`bgemm_cli`, built beside the library) as the driver of the same checks the
reference's CLI prints (lowbit_kernel/csrc/benchmark.cu:19-26 arguments, :195-218 cuBLAS fp16 yardstick, :344-350
report; shape sweeps of lowbit_kernel/run.sh:8-29). It exits non-zero unless both of its timed paths equal the
cuBLAS result element for element, so each case is one subprocess and its exit code."""
import subprocess
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu

CLI = Path(__file__).resolve().parent.parent / "bgemm-cuda_b200" / "bgemm_cli"


def _run(*args):
    assert CLI.exists(), f"{CLI} is missing: build it with `make -C {CLI.parent}`"
    r = subprocess.run([str(CLI), *map(str, args)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, f"bgemm_cli {args} exited {r.returncode}\n{r.stdout[-2000:]}\n{r.stderr[-2000:]}"
    return r.stdout


@pytest.mark.parametrize("args", [(512, 1024, 96, 0, 3),        # BWTA, automatic K partitioning
                                  (1024, 2048, 64, 4, 1),       # XOR, four K partitions
                                  (384, 1024, 32, 1, 2),        # ATTN: {0,1} mask x {-1,+1}
                                  (4096, 4096, 4, 0, 3)])       # decode shape on the weight-streaming kernel
def test_single_shape_matches_cublas(args):
    out = _run(*args)
    assert "TotalAbsError/TotalAbsSum" in out or "TotalError" in out, out[-500:]


def test_llama_sweep_matches_cublas():
    out = _run("--sweep", "llama", 32)
    assert out.count("Performance") >= 4, out[-800:]
