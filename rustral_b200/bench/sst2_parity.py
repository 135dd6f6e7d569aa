"""One-step parity check of the SST-2 classifier against an independent plain-PyTorch restatement
(scripts/eval/sst2_parity_one_step.py).

    python examples/sst2_classifier.py --overfit-32 --parity-one-step --parity-batch 8 --parity-dump out/parity.json
    python -m rustral_b200.bench.sst2_parity out/parity.json [--device cuda:0] [--atol 1e-4]

The dump holds one batch, the hyper-parameters, every parameter before the step, and what the framework computed:
logits, loss, every gradient, every parameter after one Adam step.  This module rebuilds the model from the dumped
parameters with `torch.nn.functional` only (none of the framework's layers, ops or optimizers), repeats the step with
`torch.optim.Adam`, and compares

  * the logits and the loss,
  * every gradient: maximum absolute difference, relative L2 difference, fraction of entries whose sign agrees,
  * every parameter after the step.

Exit status 0 when everything is within tolerance, 1 otherwise; the report is printed either way.
"""
from __future__ import annotations

import argparse
import json
import math
import sys

import torch
import torch.nn.functional as F


def _positions(seq: int, d: int) -> torch.Tensor:
    pos = torch.arange(seq, dtype=torch.float32).unsqueeze(1)
    div = torch.exp(torch.arange(0, d, 2, dtype=torch.float32) * (-math.log(10000.0) / d))
    pe = torch.zeros(seq, d)
    pe[:, 0::2] = torch.sin(pos * div)
    pe[:, 1::2] = torch.cos(pos * div)[:, :d // 2]
    return pe


def forward(params: dict, ids: torch.Tensor, cfg: dict) -> torch.Tensor:
    """Embedding + sinusoidal positions, `num_layers` pre-norm encoder layers (bidirectional attention without a
    padding mask, tanh GELU), final LayerNorm, mean over the non-padding positions, Linear(d, 2)."""
    d, heads, eps = cfg["d_model"], cfg["num_heads"], cfg.get("layer_norm_eps", 1e-5)
    B, S = ids.shape
    x = F.embedding(ids, params["encoder.token_embedding.embed"]) + _positions(S, d).to(ids.device)
    for i in range(cfg["num_layers"]):
        pre = f"encoder.layers.{i}."
        h = F.layer_norm(x, (d,), params[pre + "norm1.weight"], params[pre + "norm1.bias"], eps)
        q, k, v = (F.linear(h, params[pre + f"self_attn.{n}_proj.weight"], params[pre + f"self_attn.{n}_proj.bias"])
                   .view(B, S, heads, d // heads).transpose(1, 2) for n in "qkv")
        att = torch.softmax(q @ k.transpose(-1, -2) / math.sqrt(d // heads), -1) @ v
        x = x + F.linear(att.transpose(1, 2).reshape(B, S, d), params[pre + "self_attn.out_proj.weight"],
                         params[pre + "self_attn.out_proj.bias"])
        h = F.layer_norm(x, (d,), params[pre + "norm2.weight"], params[pre + "norm2.bias"], eps)
        h = F.gelu(F.linear(h, params[pre + "ff_linear1.weight"], params[pre + "ff_linear1.bias"]), approximate="tanh")
        x = x + F.linear(h, params[pre + "ff_linear2.weight"], params[pre + "ff_linear2.bias"])
    x = F.layer_norm(x, (d,), params["encoder.final_norm.weight"], params["encoder.final_norm.bias"], eps)
    keep = (ids != cfg["pad_id"]).float()
    pooled = (x * (keep / keep.sum(-1, keepdim=True).clamp_min(1.0)).unsqueeze(-1)).sum(1)
    return F.linear(pooled, params["head.weight"], params["head.bias"])


def _cmp(name: str, ours: list, theirs: torch.Tensor) -> dict:
    a = torch.tensor(ours, dtype=torch.float64)
    b = theirs.detach().double().cpu().reshape(-1)
    nz = (a != 0) | (b != 0)
    return {"name": name, "max_abs": float((a - b).abs().max()) if a.numel() else 0.0,
            "rel_l2": float((a - b).norm() / b.norm().clamp_min(1e-30)),
            "sign_agree": float((torch.sign(a[nz]) == torch.sign(b[nz])).double().mean()) if bool(nz.any()) else 1.0,
            "norm_ours": float(a.norm()), "norm_torch": float(b.norm())}


def check(dump: dict, device: str = "cpu", atol: float = 1e-4, rtol: float = 1e-3) -> dict:
    """Repeats the dumped step; returns {"ok": bool, "logits": row, "loss": (ours, torch), "grads": rows, "params": rows}."""
    cfg = dump["config"]
    params = {n: torch.tensor(v, dtype=torch.float32, device=device).view(dump["shapes"][n]).requires_grad_(True)
              for n, v in dump["params_before"].items()}
    ids = torch.tensor(dump["ids"], dtype=torch.int64, device=device)
    labels = torch.tensor(dump["labels"], dtype=torch.int64, device=device)
    logits = forward(params, ids, cfg)
    loss = F.cross_entropy(logits, labels)
    opt = torch.optim.Adam(list(params.values()), lr=cfg["lr"], betas=(cfg["adam"]["beta1"], cfg["adam"]["beta2"]), eps=cfg["adam"]["eps"])
    loss.backward()
    grads = {n: (p.grad.clone() if p.grad is not None else torch.zeros_like(p)) for n, p in params.items()}
    opt.step()
    out = {"logits": _cmp("logits", dump["logits"], logits), "loss": (dump["loss"], float(loss)), "grads": [], "params": []}
    ok = out["logits"]["max_abs"] <= atol + rtol * float(logits.abs().max()) and abs(dump["loss"] - float(loss)) <= atol + rtol * abs(float(loss))
    for n in params:
        g = dump["grads"].get(n)
        row = _cmp(n, g if g is not None else [0.0] * params[n].numel(), grads[n])
        out["grads"].append(row)
        ok = ok and row["max_abs"] <= atol + rtol * float(grads[n].abs().max())
        row = _cmp(n, dump["params_after"][n], params[n])
        out["params"].append(row)
        # one Adam step moves an entry by at most lr; where a gradient is at rounding level its sign (and so the whole
        # step) is not determined, hence the lr-sized allowance for entries whose gradient is below the tolerance
        small = grads[n].abs().reshape(-1) <= atol
        diff = (torch.tensor(dump["params_after"][n], dtype=torch.float32, device=device) - params[n].detach().reshape(-1)).abs()
        ok = ok and bool((diff[~small] <= atol + rtol * cfg["lr"] * 10).all()) and bool((diff[small] <= 2.0 * cfg["lr"] + atol).all())
    out["ok"] = bool(ok)
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="rustral_b200.bench.sst2_parity")
    ap.add_argument("dump")
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--atol", type=float, default=1e-4)
    ap.add_argument("--rtol", type=float, default=1e-3)
    a = ap.parse_args(argv)
    with open(a.dump) as f:
        dump = json.load(f)
    res = check(dump, a.device, a.atol, a.rtol)
    print(f"loss: framework {res['loss'][0]:.7f}  torch {res['loss'][1]:.7f}")
    print(f"logits: max|diff| {res['logits']['max_abs']:.3e}  rel L2 {res['logits']['rel_l2']:.3e}")
    print(f"{'gradient':<44} {'max|diff|':>10} {'rel L2':>10} {'sign ok':>8} {'|g| ours':>11} {'|g| torch':>11}")
    for r in res["grads"]:
        print(f"{r['name']:<44} {r['max_abs']:>10.3e} {r['rel_l2']:>10.3e} {r['sign_agree']:>8.4f} {r['norm_ours']:>11.4e} {r['norm_torch']:>11.4e}")
    worst = max(res["params"], key=lambda r: r["max_abs"])
    print(f"parameters after one Adam step: worst max|diff| {worst['max_abs']:.3e} ({worst['name']})")
    print("PARITY OK" if res["ok"] else "PARITY FAILED")
    return 0 if res["ok"] else 1


if __name__ == "__main__":
    sys.exit(main())
