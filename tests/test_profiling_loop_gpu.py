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


@pytest.mark.parametrize("task,model_dir,env", [("gdn", "gdn", {"CAB_GDN_CONFIG": "0"}),
                                                ("mla", "mla", {"CAB_MLA_CONFIG": "1"}),
                                                ("moe", "moe", {"CAB_MOE_CONFIG": "0"}),
                                                ("moe_ep", "moe", {"CAB_MOE_CONFIG": "1"})])
def test_three_column_line_for_every_task(cuda_device, built_libs, capsys, task, model_dir, env):
    """Eager, torch.compile and extension columns (the reference's full line, utils/profiling.py:76-82) for
    each task on its small configuration."""
    os.environ.update(env)
    sys.path.insert(0, str(built_libs.WORKDIR))
    from utils import profiling
    args = ["--task", str(built_libs.WORKDIR / "tasks" / task), "--model-dir", str(ROOT / "oracle" / model_dir)]
    assert profiling.main(args + ["--iters", "3"]) == 0
    out = capsys.readouterr().out
    m = re.search(r"Torch Baseline: ([\d.]+)us, Torch Compile: ([\d.]+)us, CUDA Extension: ([\d.]+)us", out)
    assert m, out
    assert all(float(g) > 0 for g in m.groups())
