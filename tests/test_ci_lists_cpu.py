"""The tier lists a CI job consumes must name every test file exactly where its markers put it."""
import glob
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
GPU_MARK = "pytest.mark." + "gpu"        # spelt in two parts so that this file does not match itself
MULTI_MARK = "mark." + "multigpu"


def _listed(tier):
    with open(os.path.join(HERE, f"ci_test_list_{tier}.txt")) as f:
        return {line.strip() for line in f if line.strip() and not line.startswith("#")}


def test_every_test_file_is_in_the_tier_lists_its_markers_imply():
    cpu, gpu, multi = _listed("cpu"), _listed("gpu"), _listed("multigpu")
    for path in sorted(glob.glob(os.path.join(HERE, "test_*.py"))):
        rel = "tests/" + os.path.basename(path)
        src = open(path).read()
        module_gpu = re.search(r"^pytestmark\s*=.*gpu", src, re.M) is not None
        assert (rel in gpu) == (GPU_MARK in src), rel
        assert (rel in multi) == (MULTI_MARK in src), rel
        assert (rel in cpu) == (not module_gpu), rel
    for rel in cpu | gpu | multi:
        assert os.path.exists(os.path.join(os.path.dirname(HERE), rel)), rel
