"""The kernels built with their index checks (FMS_B200_DEBUG_BOUNDS=1, csrc/common.cuh): the stand-in for a memory
checker.  Each case runs in a process of its own with the flag set, so that the checked libraries are the ones
loaded; they are compiled at first use, beside the ordinary ones.

1. An index outside its array is recorded with its source line, index and extent, the access is skipped, nothing
   traps and the process goes on.  The case is made so that not even an unchecked kernel would leave allocated
   memory: the kernel is told that the cache has 4 blocks while the storage behind it has 8, and a table entry
   names block 6.
2. A tiny model generates through the entry point and equals the plain implementation, with no index recorded.
3. The kernel tests run under the flag (small cases: the slowest, many-sequence ones are left out); a fixture in
   conftest.py fails any of them that records an index.
"""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ENV = dict(os.environ, FMS_B200_DEBUG_BOUNDS="1")

RECORDS_AND_SKIPS = r'''
import sys, torch
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, sys.argv[1] + "/tests")
from fms_b200.kernels import build, ops
assert build.DEBUG_BOUNDS
from fms_b200.cache.cache import KVLayerView
from fms_b200.engine.batch import Batch

nheads, kvheads, hd = 2, 1, 16
storage = torch.zeros(2, 8, kvheads, 64, hd, device="cuda")          # 8 blocks are really there
view = KVLayerView(storage[0, :4], storage[1, :4], torch.tensor([[1, 6]], dtype=torch.int32, device="cuda"), 0)  # 4 are declared
batch = Batch.from_lists([0], [60], [[0] * 8], [[]], "cuda")           # positions 60..67: blocks 1 and 6 of the table
qkv = torch.ones(8, (nheads + 2 * kvheads) * hd, device="cuda")
q = ops.rope_store(qkv, None, batch, view, nheads, kvheads, hd)
try:
    ops.check_error_flag("cuda")
    raise SystemExit("nothing was recorded")
except ops.KernelError as e:
    text = str(e)
    assert "index 6, extent 4" in text and "elementwise" in text, text
assert float(storage[:, 6].abs().sum()) == 0.0          # the access was skipped
assert float(storage[0, 1, 0, 60:].sum()) == 4 * hd      # the rows inside the cache were written
ops.check_error_flag("cuda")                              # the record was cleared by reading it
print("recorded and skipped")
'''

GENERATES = r'''
import sys, tempfile, torch
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, sys.argv[1] + "/tests")
from fms_b200.kernels import build
assert build.DEBUG_BOUNDS
import plain_llama as pl
from tiny_models import tiny_prompts, write_tiny
from fms_b200.models import get_model
from fms_b200.utils.generation import generate
folder = write_tiny(tempfile.mkdtemp(), "d")
oracle = pl.PlainLlama(folder)
prompts = tiny_prompts("d")
for dtype in ("fp32", "bf16"):
    model = get_model("hf_pretrained", model_path=folder, device_type="cuda", data_type=dtype)
    out = generate(model, [torch.tensor(p) for p in prompts], max_new_tokens=6, do_sample=False)
    model.engine().check()
    if dtype == "fp32":
        assert [o.tolist() for o in out] == [pl.plain_generate(oracle, p, 6) for p in prompts]
assert build.bounds_violations() == []
assert all("_checked_" in lib._name for lib in build.loaded_libraries().values())
print("generated")
'''


def _run(code):
    return subprocess.run([sys.executable, "-c", code, ROOT], env=ENV, capture_output=True, text=True, timeout=1500)


@pytest.mark.expects_a_recorded_index
def test_an_index_outside_its_array_is_recorded_and_skipped():
    r = _run(RECORDS_AND_SKIPS)
    assert r.returncode == 0 and "recorded and skipped" in r.stdout, (r.stdout + r.stderr)[-3000:]


def test_a_model_generates_under_the_index_checks():
    r = _run(GENERATES)
    assert r.returncode == 0 and "generated" in r.stdout, (r.stdout + r.stderr)[-3000:]


def test_the_kernel_tests_pass_under_the_index_checks():
    r = subprocess.run([sys.executable, "-m", "pytest", os.path.join(ROOT, "tests", "test_kernels_gpu.py"), "-q", "-x", "-m", "gpu",
                        "-k", "not streams_the_cache and not every_batch_size and not 128256 and not long_context"],
                       env=ENV, capture_output=True, text=True, timeout=3000, cwd=ROOT)
    assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
