"""Child process of tests/test_gpu_bounds.py: runs with RUSTRAL_BOUNDS=1, i.e. on the index-checking build of the kernel
library, feeds each index-reading kernel one out-of-range index and reads the report from the status word.  The kernels
skip or clamp such an index in every build (nothing is dereferenced out of range); this build also says so."""
import json
import math
import sys

import torch

from rustral_b200 import _native as N
from rustral_b200 import ops
from rustral_b200.ops import paged

lib = N.kernels()
assert N.KERNEL_LIB == "librb200_kernels_bounds.so" and lib.rb_build_flags() & 1, "not the checking build"
lib.rb_init()
N.read_status(clear=True)
dev = "cuda"
out = {}


def status():
    torch.cuda.synchronize()
    bits, where = N.read_status(clear=True)
    return [int(bits), int(where)]


g = torch.Generator().manual_seed(0)
wte = torch.randn(50, 64, generator=g).bfloat16().to(dev)
ids = torch.tensor([[1, 2, 3, 4]], device=dev)
y = ops.embedding_forward(ids, wte)
out["embedding_ok"] = status()
bad = ids.clone(); bad[0, 2] = 50
y2 = ops.embedding_forward(bad, wte)
out["embedding_bad"] = status()
out["embedding_bad_reads_row0"] = bool(torch.equal(y2.view(-1, 64)[2], wte[0]) and torch.equal(y2.view(-1, 64)[3], y.view(-1, 64)[3]))

a = torch.randn(10, 16, generator=g).to(dev)
r = ops.gather_rows(a, torch.tensor([0, 9, 3], device=dev))
out["gather_ok"] = status()
r2 = ops.gather_rows(a, torch.tensor([0, 10, 3], device=dev))
out["gather_bad"] = status()
out["gather_bad_row_is_zero"] = bool((r2[1] == 0).all() and torch.equal(r2[2], a[3]))

logits = torch.randn(4, 32, generator=g).bfloat16().to(dev)
tgt = torch.tensor([1, 5, 31, -100], device=dev)
ops.cross_entropy_fwd_bwd(logits, tgt, 32, 1.0)
out["ce_ok"] = status()
ops.cross_entropy_fwd_bwd(logits, torch.tensor([1, 32, 2, -100], device=dev), 32, 1.0)
out["ce_bad"] = status()

nb, bs, hk, d = 4, 16, 2, 64
kc = torch.zeros(nb, bs, hk, d, dtype=torch.bfloat16, device=dev)
vc = torch.zeros_like(kc)
kn = torch.randn(3, hk * d, generator=g).bfloat16().to(dev)
paged.kv_append(kn, kn, kc, vc, torch.tensor([0, -1, 5], device=dev))
out["kv_ok"] = status()
paged.kv_append(kn, kn, kc, vc, torch.tensor([0, nb * bs, 5], device=dev))
out["kv_bad"] = status()

q = torch.randn(1, 4 * d, generator=g).bfloat16().to(dev)
bt = torch.tensor([[1, 2]], dtype=torch.int32, device=dev)
ctx = torch.tensor([20], dtype=torch.int32, device=dev)
paged.paged_attention_decode(q, kc, vc, bt, ctx, 1 / math.sqrt(d))
out["paged_ok"] = status()
paged.paged_attention_decode(q, kc, vc, torch.tensor([[1, 7]], dtype=torch.int32, device=dev), ctx, 1 / math.sqrt(d))
out["paged_bad"] = status()

# an ordinary small training step on this build leaves the status word clean
from rustral_b200.models.config import preset
from rustral_b200.runtime.lm_trainer import LMTrainer, TrainConfig
cfg = preset("gpt2-test", seq_len=64)
tr = LMTrainer(cfg, TrainConfig(global_batch=4, micro_batch=2), torch.device(dev))
toks = torch.randint(0, cfg.vocab_size, (4, 65), generator=g)
out["loss"] = tr.step(toks)
out["train_step"] = status()
print(json.dumps(out))
