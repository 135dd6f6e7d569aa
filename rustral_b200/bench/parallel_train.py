"""Training-throughput benchmark of the parallel decoder LM: tensor parallel (fused or over collectives), tensor x
pipeline parallel (1F1B) and expert parallel, one rank per GPU under torch.distributed.run.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29700 \
        -m rustral_b200.bench.parallel_train --config llama-8b --tp 8 --global-batch 64 --micro-batch 1
    ... --config llama-8b --tp 4 --pp 2 --global-batch 64 --micro-batch 8          (8 micro-batches, 1F1B)
    ... --config moe-24l --ep 8 --global-batch 128 --micro-batch 4
    ... --config llama-8b --cp 8 --seq 65536 --global-batch 1 --micro-batch 1      (context parallel, 8192 tokens per GPU)
    add --unfused for the same run over NCCL collectives (tensor parallel) as the comparison arm

Synthetic data (uniform random token ids from a seed), random-init weights, AdamW with fp32 master weights.
Device-timed with CUDA events over `--steps` optimizer steps after `--warmup`, max over ranks; rank 0 prints JSON.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist


def build_config(name: str, layers: int, seq: int):
    from ..models.parallel_lm import ParallelLMConfig, llama_8b, moe_24l
    kw = {}
    if layers:
        kw["n_layer"] = layers
    if seq:
        kw["seq_len"] = seq
    if name == "llama-8b":
        return llama_8b(**kw)
    if name == "moe-24l":
        return moe_24l(**kw)
    if name == "tiny":
        base = dict(vocab_size=1024, d_model=256, n_layer=4, n_head=4, n_kv_head=2, ffn_hidden=512, seq_len=256)
        base.update(kw)
        return ParallelLMConfig(**base)
    if name == "tiny-moe":
        base = dict(vocab_size=1024, d_model=256, n_layer=2, n_head=4, n_kv_head=4, ffn_hidden=256, seq_len=256,
                    num_experts=4, top_k=2)
        base.update(kw)
        return ParallelLMConfig(**base)
    raise SystemExit(f"unknown config {name}")


def main(argv=None):
    ap = argparse.ArgumentParser(prog="rustral_b200.bench.parallel_train")
    ap.add_argument("--config", default="tiny")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--pp", type=int, default=1)
    ap.add_argument("--ep", type=int, default=1)
    ap.add_argument("--fsdp", type=int, default=1, help="data-parallel ranks with ZeRO-3 sharded block weights (fused all-gather)")
    ap.add_argument("--cp", type=int, default=1, help="context-parallel ranks: every sequence is split over them (ring attention "
                    "over NVLink peer memory)")
    ap.add_argument("--cp-contiguous", action="store_true", help="contiguous instead of striped token assignment")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--seq", type=int, default=0)
    ap.add_argument("--global-batch", type=int, default=8)
    ap.add_argument("--micro-batch", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--lr", type=float, default=3e-4)
    ap.add_argument("--capacity-factor", type=float, default=1.5, help="expert-parallel receive capacity (x balanced share)")
    ap.add_argument("--init-from", help="safetensors checkpoint (unsharded, this framework's names; see utils.hf for "
                    "Hugging Face conversion): every rank loads its shard instead of the random initialisation")
    ap.add_argument("--save-dir", help="after training, write the unsharded checkpoint (dense models): one file per pipeline "
                    "stage (stage<k>.safetensors, reassembled over the tensor-parallel ranks); their union is the model")
    ap.add_argument("--unfused", action="store_true")
    ap.add_argument("--same-batch", action="store_true", help="train on one fixed batch (tests: the loss must fall)")
    a = ap.parse_args(argv)

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if a.ep > 1 and (a.tp > 1 or a.pp > 1):
        raise SystemExit("expert parallelism is combined with data parallelism only")
    if a.fsdp > 1 and (a.tp > 1 or a.pp > 1 or a.ep > 1):
        raise SystemExit("--fsdp is combined with plain data parallelism only")
    if a.cp > 1 and (a.tp > 1 or a.pp > 1 or a.ep > 1 or a.fsdp > 1):
        raise SystemExit("--cp is combined with plain data parallelism only")
    if a.tp * a.pp * a.ep * a.fsdp * a.cp != world:
        raise SystemExit(f"tp*pp*ep*fsdp*cp = {a.tp * a.pp * a.ep * a.fsdp * a.cp} but WORLD_SIZE = {world}")

    from .. import _native
    from ..models.parallel_lm import MixedPrecisionAdamW, ParallelDecoderLM
    from ..parallel.process_group import ProcessGroup
    cfg = build_config(a.config, a.layers, a.seq)
    S = cfg.seq_len

    tp_pg = pp_pg = None
    fused_tp = ep_ctx = None
    tp_idx, pp_idx = (rank % a.tp, rank // a.tp) if (a.ep == 1 and a.fsdp == 1 and a.cp == 1) else (0, 0)
    cp_ctx = None
    if a.cp > 1:
        from ..parallel.peer_ring import PeerRing
        cp_ctx = PeerRing(dist.group.WORLD, dev, a.micro_batch * (S // a.cp) * cfg.n_kv_head * cfg.head_dim)
    fsdp_ctx = None
    if a.fsdp > 1:
        from ..parallel.fused_tp import FusedTP
        fsdp_ctx = FusedTP(None, dev)
    if a.tp > 1:
        for p in range(a.pp):                                  # every rank takes part in creating every group
            g = ProcessGroup.new_torch_subgroup(range(p * a.tp, (p + 1) * a.tp))
            if p == pp_idx:
                tp_pg = g
        if not a.unfused:
            from ..parallel.fused_tp import FusedTP
            fused_tp = FusedTP(tp_pg.group, dev)
    if a.pp > 1:
        for t in range(a.tp):
            g = ProcessGroup.new_torch_subgroup(range(t, world, a.tp))
            if t == tp_idx:
                pp_pg = g
    if a.ep > 1:
        from ..parallel.expert_parallel import FusedEP
        ep_ctx = FusedEP(None, dev, cfg.num_experts, cfg.d_model, max_tokens=a.micro_batch * S, k=cfg.top_k,
                         capacity_factor=a.capacity_factor if a.capacity_factor > 0 else None)

    per_stage = cfg.n_layer // a.pp
    model = ParallelDecoderLM(cfg, dev, tp_pg=tp_pg, fused_tp=fused_tp, ep=ep_ctx,
                              first_layer=pp_idx * per_stage, last_layer=(pp_idx + 1) * per_stage if pp_idx < a.pp - 1 else cfg.n_layer,
                              has_embed=pp_idx == 0, has_head=pp_idx == a.pp - 1, seed=1, fsdp=fsdp_ctx,
                              cp=cp_ctx, cp_striped=not a.cp_contiguous, dp_group=dist.group.WORLD if cp_ctx is not None else None)
    if a.init_from:
        from ..io import safetensors_io as st
        model.load_state_dict(st.load_file(a.init_from)[0])
    # expert parallel: ZeRO-1 over the data-parallel ranks for the dense (replicated) parameters
    opt = MixedPrecisionAdamW(model, lr=a.lr, use_zero1=a.ep > 1)
    dp = a.ep * a.fsdp                                         # data-parallel replicas (these ranks see different data)
    local_batch = a.global_batch // dp
    if local_batch % a.micro_batch:
        raise SystemExit("the per-replica batch must be a multiple of the micro-batch")
    n_micro = local_batch // a.micro_batch

    pipe = None
    if a.pp > 1:
        from ..parallel.pipeline_parallel import PipelineConfig, PipelineParallel, PipelineSchedule, PipelineStage

        def fwd(x):
            if pp_idx == 0:
                x = model.embed(x[:, :-1])
            y, _ = model.blocks(x, a.micro_batch, S)
            return y

        stage = PipelineStage(pp_idx, a.pp, fwd, model.parameters())
        pipe = PipelineParallel(stage, pp_pg, PipelineConfig(num_micro_batches=n_micro, schedule=PipelineSchedule.INTERLEAVED),
                                act_shape=(a.micro_batch * S // a.tp, cfg.d_model), act_dtype=torch.bfloat16, device=dev)
        pipe.after_backward = opt.accumulate

    gen = torch.Generator().manual_seed(1234 + (rank if dp > 1 else 0))     # TP / PP ranks of a replica see the same batch

    def make_batch():
        return torch.randint(0, cfg.vocab_size, (local_batch, S + 1), generator=gen, dtype=torch.int64).to(dev)

    def train_step(tokens):
        mbs = [tokens[i * a.micro_batch:(i + 1) * a.micro_batch] for i in range(n_micro)]
        if pipe is not None:
            loss = pipe.train_step(inputs=mbs, targets=[m[:, 1:] for m in mbs], loss_fn=lambda y, t: model.loss(y, t))
        else:
            total = None
            for m in mbs:
                loss_mb = model.forward_loss(m) / n_micro
                loss_mb.backward()
                opt.accumulate()
                total = loss_mb.detach() if total is None else total + loss_mb.detach()
            loss = total
        opt.step()
        return loss

    batches = [make_batch() for _ in range(a.warmup + a.steps)]
    if a.same_batch:
        batches = [batches[0]] * len(batches)
    losses = []
    for i in range(a.warmup):
        losses.append(train_step(batches[i]))
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(a.steps):
        losses.append(train_step(batches[a.warmup + i]))
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / a.steps], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    status = torch.tensor([_native.read_status()[0]], device=dev)
    if world > 1:
        dist.all_reduce(status, op=dist.ReduceOp.MAX)
    # the loss lives on the last pipeline stage
    loss_vals = [float(l) if l is not None else float("nan") for l in losses]
    lt = torch.tensor(loss_vals, dtype=torch.float64, device=dev)
    if world > 1 and a.pp > 1:
        lt = torch.nan_to_num(lt, nan=0.0)
        dist.all_reduce(lt, op=dist.ReduceOp.MAX)
    if a.cp > 1:                                               # every rank holds the mean over ITS tokens
        dist.all_reduce(lt)
        lt /= world
    tokens = a.global_batch * S
    if rank == 0:
        ms_step = float(ms)
        print(json.dumps({
            "metric": "train_tokens_per_s", "value": round(tokens / (ms_step / 1e3), 1), "unit": "tokens/s",
            "n_gpus": world, "ms_per_step": round(ms_step, 2), "steps": a.steps, "warmup": a.warmup, "dtype": "bf16",
            "config": {"model": a.config, "layers": cfg.n_layer, "d_model": cfg.d_model, "seq_len": S,
                       "global_batch": a.global_batch, "micro_batch": a.micro_batch,
                       "parallelism": f"tp{a.tp}-pp{a.pp}-ep{a.ep}" + (f"-fsdp{a.fsdp}" if a.fsdp > 1 else "") +
                                      (f"-cp{a.cp}{'c' if a.cp_contiguous else 's'}" if a.cp > 1 else ""),
                       "fused": not a.unfused,
                       "params_total": cfg.num_params(), "params_local": model.local_param_count(),
                       "zero1_dense": a.ep > 1, "optimizer_state_bytes_local": opt.state_bytes()},
            "model_tflops_per_s_per_gpu": round(cfg.flops_per_token() * tokens / (ms_step / 1e3) / 1e12 / world, 1),
            "losses": [round(v, 4) for v in lt.tolist()], "device_status": int(status),
            "data": "synthetic (uniform random token ids), random-init weights"}))
    if a.save_dir and not cfg.num_experts and a.fsdp == 1:
        from ..io import safetensors_io as st
        state = model.gather_state_dict()                      # collective over the tensor-parallel group
        writes = tp_idx == 0 and (a.pp > 1 or a.tp > 1 or rank == 0)
        if writes:
            os.makedirs(a.save_dir, exist_ok=True)
            st.save_file(state, os.path.join(a.save_dir, f"stage{pp_idx}.safetensors"),
                         {"layers": f"{model.first_layer}-{model.last_layer}", "config": a.config})
    if world > 1:
        dist.barrier()
    if fused_tp is not None:
        fused_tp.close()
    if ep_ctx is not None:
        ep_ctx.close()
    if fsdp_ctx is not None:
        fsdp_ctx.close()
    if cp_ctx is not None:
        cp_ctx.close()
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
