"""The index-checking build (-DCLT_DEBUG_BOUNDS): a training step runs clean under it, and an entry whose feature index lies
outside the decoder is reported through the status word while its access is skipped (the regular build trusts its lists)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SCRIPT = r'''
import sys, torch
sys.path.insert(0, %r)
from crosslayer_coding_b200 import CLTConfig, CrossLayerTranscoder, TrainingConfig
from crosslayer_coding_b200.ops import ext
from crosslayer_coding_b200.training.fused_engine import FusedBatchTopKEngine, EngineStatusError
e = ext.load()
assert e.__name__.endswith("_dbg"), e.__name__
dev = torch.device("cuda:0")
torch.manual_seed(0)
L, B, d, F = 3, 128, 64, 256
cfg = CLTConfig(num_features=F, num_layers=L, d_model=d, activation_fn="batchtopk", batchtopk_k=6, clt_dtype="bfloat16")
model = CrossLayerTranscoder(cfg, device=dev)
tc = TrainingConfig(learning_rate=1e-3, training_steps=10, activation_path="unused", precision="bf16", sparsity_lambda=0.01, preactivation_coef=0.0)
eng = FusedBatchTopKEngine(model, tc, B)
X = torch.randn(L, B, d, device=dev).bfloat16()
Y = torch.randn(L, B, d, device=dev).bfloat16()
for step in range(3):
    out = eng.train_step(X, Y, step, 1e-3, sparsity_lambda=0.01)
torch.cuda.synchronize()
eng.check_status()                       # no index complaint on a regular step
# an entry that names feature F (one past the last): the debug build reports it and leaves the row untouched
eng.encode_select(X)
torch.cuda.synchronize()
eng.tcsr_col[0] = (1 << 24) | F
eng.decode_loss(Y)
torch.cuda.synchronize()
try:
    eng.check_status()
    print("NO-REPORT")
except EngineStatusError as exc:
    print("REPORTED", exc)
'''


def test_debug_build_runs_clean_and_reports_a_bad_entry():
    env = dict(os.environ, CLT_DEBUG_BOUNDS="1")
    res = subprocess.run([sys.executable, "-c", SCRIPT % REPO], env=env, capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
    assert "REPORTED" in res.stdout and "index out of range" in res.stdout and "value 256" in res.stdout, res.stdout[-1000:]
