"""The workspace builds the way the reference builds its own (one torch.utils.cpp_extension.load over
*.cu / *.cpp in the root and kernels/, agent_workdir/utils/compile.py:11-50), with sm_100a from
TORCH_CUDA_ARCH_LIST; no GPU needed."""
import os
import shutil
import subprocess
import sys

from conftest import ROOT


def test_reference_style_single_load_build(tmp_path):
    wd = tmp_path / "agent_workdir"
    shutil.copytree(ROOT / "cuda_agent_b200" / "agent_workdir", wd,
                    ignore=shutil.ignore_patterns("*.so", "build", "__pycache__"))
    (tmp_path / "include").mkdir()
    shutil.copy(ROOT / "include" / "cuda_agent_b200.h", tmp_path / "include")
    for name in ("cab_common.cuh", "binding_common.h"):
        f = wd / "kernels" / name
        f.write_text(f.read_text().replace("../../../include/cuda_agent_b200.h", "../../include/cuda_agent_b200.h"))
    env = dict(os.environ, TORCH_CUDA_ARCH_LIST="10.0a")
    out = subprocess.run(["bash", "utils/compile.sh", "--torch-load"], cwd=wd, env=env, capture_output=True,
                         text=True, timeout=900)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "Compile success: cuda_extension.so" in out.stdout and "[TIME] Compilation took" in out.stdout
    probe = subprocess.run([sys.executable, "-c",
                            "import torch, cuda_extension as e; print(sorted(e.registered_ops()))"],
                           cwd=wd, capture_output=True, text=True, timeout=300)
    assert probe.returncode == 0, probe.stderr
    assert "['axpby', 'gdn_decode', 'mla', 'moe', 'moe_ep']" in probe.stdout
