"""The reference-style timing loop (utils/profiling.py) on the GPU: result line and --single-run."""
import os
import re
import sys

import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu


def test_profiling_loop_prints_the_reference_line(cuda_device, built_libs, capsys):
    os.environ["CAB_GDN_CONFIG"] = "0"
    sys.path.insert(0, str(built_libs.WORKDIR))
    from utils import profiling
    args = ["--task", str(built_libs.WORKDIR / "tasks" / "gdn"), "--model-dir", str(ROOT / "oracle" / "gdn")]
    assert profiling.main(args + ["--iters", "5", "--no-compile", "--events"]) == 0
    out = capsys.readouterr().out
    m = re.search(r"Torch Baseline: ([\d.]+)us, Torch Compile: (nan|[\d.]+)us, CUDA Extension: ([\d.]+)us", out)
    assert m, out
    assert float(m.group(3)) > 0 and float(m.group(1)) > float(m.group(3))     # one kernel beats the eager chain
    assert profiling.main(args + ["--single-run", "torch_baseline,cuda_extension"]) == 0
    assert "[DONE] single-run completed" in capsys.readouterr().out
