"""The kernels' bounds-check build (-DLLM_BOUNDS_CHECK): an out-of-range page id is reported through a status word and the
access is redirected into the allocation, instead of faulting the GPU.  Runs in a child process because the variant is a
separate build of the extension (its own directory), selected by LLAMINAR_BOUNDS_CHECK before the first import."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

CHILD = r'''
import math, torch
from llaminar_b200 import ops
assert ops.ext().bounds_check_build
dev = "cuda"
B, nq, nkv, D, pages = 2, 4, 2, 128, 4
kv = (torch.randn(9, 2, nkv, 64, D, device=dev) * 0.3).to(torch.bfloat16)
q = (torch.randn(B, nq, D, device=dev) * 0.3).to(torch.bfloat16)
out = torch.empty_like(q)
lens = torch.full((B,), 100, dtype=torch.int32, device=dev)
sc = ops.scratch_for(dev)
good = torch.tensor([[1, 2, 0, 0], [3, 4, 0, 0]], dtype=torch.int32, device=dev)
ops.attn_decode(q, kv, out, good, lens, nq, nkv, D, 1, 1.0 / math.sqrt(D), 1, sc)
torch.cuda.synchronize()
assert ops.bounds_status() == 0
bad = good.clone()
bad[1, 1] = 1_000_000                      # far outside the 9 pages of the cache
ops.attn_decode(q, kv, out, bad, lens, nq, nkv, D, 1, 1.0 / math.sqrt(D), 1, sc)
torch.cuda.synchronize()                   # no fault: the kernel read page 0 instead
assert ops.bounds_status() == 3            # STATUS_BAD_INDEX, and the word is cleared by the read
assert ops.bounds_status() == 0
qkv = (torch.randn(B, (nq + 2 * nkv) * D, device=dev) * 0.3).to(torch.bfloat16)
qo = torch.empty(B, nq, D, dtype=torch.bfloat16, device=dev)
pos = torch.tensor([70, 71], dtype=torch.int32, device=dev)
sid = torch.tensor([0, 1], dtype=torch.int32, device=dev)
ops.rope_kv(qkv, qo, kv, None, None, pos, sid, bad, nq, nkv, D, 1e6, 1e-6)
torch.cuda.synchronize()
assert ops.bounds_status() == 3            # the KV append was redirected to page 0 and reported
print("BOUNDS_CHECK_OK")
'''


def test_bounds_check_build_reports_a_bad_page_id_instead_of_faulting():
    env = dict(os.environ, LLAMINAR_BOUNDS_CHECK="1")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", CHILD], cwd=root, env=env, capture_output=True, text=True, timeout=1500)
    assert "BOUNDS_CHECK_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]
