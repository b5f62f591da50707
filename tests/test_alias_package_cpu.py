"""``import fastdeploy`` gives the same modules as ``import fastdeploy_b200`` (checked in a child process so that this
session's module table stays as it is)."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

PROGRAM = r"""
import fastdeploy as fd
import fastdeploy_b200 as real
assert fd is real and fd.__version__ == real.__version__
import fastdeploy.vision.detection as det
from fastdeploy.vision.detection import PPYOLOE
from fastdeploy.vision.common.manager import PyProcessorManager
from fastdeploy.vision.common.processors import ResizeByShort
from fastdeploy.runtime import Runtime, RuntimeOption
from fastdeploy.model import FastDeployModel
from fastdeploy import c_lib_wrap as C
import fastdeploy.text, fastdeploy.serving, fastdeploy.encryption, fastdeploy.pipeline, fastdeploy.download
import fastdeploy_b200.vision.detection as real_det
assert det is real_det and PPYOLOE is real_det.PPYOLOE
assert Runtime is real.Runtime and RuntimeOption is real.RuntimeOption and FastDeployModel is real.FastDeployModel
assert C.vision.DetectionResult is real.vision.DetectionResult
assert issubclass(PPYOLOE, FastDeployModel)
import sys
assert sys.modules["fastdeploy.vision"] is sys.modules["fastdeploy_b200.vision"]
try:
    import fastdeploy.no_such_module
except ModuleNotFoundError:
    pass
else:
    raise SystemExit("a missing module must stay missing")
opt = fd.RuntimeOption(); opt.use_cpu()
print("ok", fd.vision.DetectionResult().__class__.__module__)
"""


def test_alias_package_shares_module_objects():
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    p = subprocess.run([sys.executable, "-c", PROGRAM], capture_output=True, text=True, env=env, cwd=ROOT, timeout=300)
    assert p.returncode == 0, p.stdout + p.stderr
    assert p.stdout.strip().splitlines()[-1] == "ok fastdeploy_b200.vision.result"
