"""A process that drives several GPUs: per-device kernel attributes and per-device state must be set up
on whichever device is used first (the reference's PyTorch path spreads a model with device_map="auto",
src/utils.py:60).  Each case runs in a fresh interpreter so that device 1 really is the first one used."""
from __future__ import annotations

import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_FIRST_CALL_ON_DEVICE_1 = r"""
import sys
sys.path.insert(0, %r)
import torch
import tidaldecode_b200.ops as T
from oracle import tidal_oracle as O
torch.cuda.set_device(1)
g = torch.Generator().manual_seed(4)
s = torch.randn(3, 40000, generator=g)
ws = T.Workspace(1, 1, 64, 3, 40000, device="cuda:1")
idx = T.topk(s.to("cuda:1"), 256, ws)          # the cluster kernel: more dynamic shared memory than the default limit
torch.cuda.synchronize()
ok, why = O.topk_sets_match(s, idx.cpu(), 256, tie_band=0.0)
assert ok, why
assert ws.status() == 0
torch.cuda.set_device(0)
ws0 = T.Workspace(1, 1, 64, 3, 40000, device="cuda:0")
idx0 = T.topk(s.to("cuda:0"), 256, ws0)
torch.cuda.synchronize()
assert torch.equal(idx0.cpu(), idx.cpu())
print("ok")
"""


def test_topk_first_call_on_second_device():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    r = subprocess.run([sys.executable, "-c", _FIRST_CALL_ON_DEVICE_1 % ROOT], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout + r.stderr
