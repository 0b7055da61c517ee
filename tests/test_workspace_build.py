"""The workspace builds the way the reference builds its own (one torch.utils.cpp_extension.load over
*.cu / *.cpp in the root and kernels/, agent_workdir/utils/compile.py:11-50), with sm_100a from
TORCH_CUDA_ARCH_LIST; no GPU needed."""
import os
import shutil
import subprocess
import sys

from conftest import ROOT


import pytest


def export_and_build(tmp_path, task):
    """A self-contained workspace for `task`, built the reference's way (utils/compile.sh from inside it)."""
    from cuda_agent_b200 import export_task
    wd = export_task.export(task, tmp_path / f"agent_workdir_{task}")
    for name in ("model.py", "model_new.py", "SKILL.md", "binding.cpp", "binding_registry.h", "TASK_CONFIG.env",
                 "kernels/gdn_decode.cu", "utils/verification.py", "include/cuda_agent_b200.h"):
        assert (wd / name).exists(), name
    env = dict(os.environ, TORCH_CUDA_ARCH_LIST="10.0a")
    out = subprocess.run(["bash", "utils/compile.sh"], cwd=wd, env=env, capture_output=True, text=True, timeout=1200)
    return wd, out


def test_reference_style_single_load_build(tmp_path):
    wd, out = export_and_build(tmp_path, "gdn")
    assert out.returncode == 0, out.stdout + out.stderr
    assert "Compile success: cuda_extension.so" in out.stdout and "[TIME] Compilation took" in out.stdout
    probe = subprocess.run([sys.executable, "-c",
                            "import torch, cuda_extension as e; print(sorted(e.registered_ops()))"],
                           cwd=wd, capture_output=True, text=True, timeout=300)
    assert probe.returncode == 0, probe.stderr
    assert "['axpby', 'gdn_decode', 'mla', 'moe', 'moe_ep']" in probe.stdout


@pytest.mark.gpu
def test_exported_task_workspace_verifies_by_cd_alone(tmp_path):
    """The reference's loop on a directory of its own: export, cd, compile, verify, time."""
    wd, out = export_and_build(tmp_path, "mla")
    assert out.returncode == 0, out.stdout + out.stderr
    env = dict(os.environ)
    key, val = (wd / "TASK_CONFIG.env").read_text().strip().split("=")
    env[key] = val
    ver = subprocess.run([sys.executable, "-m", "utils.verification"], cwd=wd, env=env, capture_output=True, text=True,
                         timeout=600)
    assert ver.returncode == 0 and "[PASS] verify success" in ver.stdout, ver.stdout + ver.stderr
    prof = subprocess.run([sys.executable, "-m", "utils.profiling", "--iters", "3", "--no-compile"], cwd=wd, env=env,
                          capture_output=True, text=True, timeout=600)
    assert prof.returncode == 0 and "CUDA Extension:" in prof.stdout, prof.stdout + prof.stderr
