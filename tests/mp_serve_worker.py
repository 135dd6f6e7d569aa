"""Worker for the tensor-parallel serving test: every rank serves its shard of a small Llama-style model and compares
prefill and decode logits with the unsharded model run on the same GPU.  Rank 0 prints one JSON line."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    from rustral_b200 import _native
    from rustral_b200.models.config import GPTConfig
    from rustral_b200.parallel.tp_inference import TPInferenceComm
    from rustral_b200.runtime.fused_gpt import FlatParams
    from rustral_b200.serve.engine import ServingEngine
    from rustral_b200.serve.model_runner import ModelRunner
    from rustral_b200.serve.weights import InferenceWeights
    cfg = GPTConfig(vocab_size=1000, seq_len=512, n_layer=2, n_head=4, n_kv_head=2, d_model=256, ffn_dim=512, arch="llama",
                    vocab_multiple=128)
    full = FlatParams(cfg, dev, seed=3)                       # the same on every rank
    tp = TPInferenceComm(None, dev, max_elems=512 * 1024, transport=os.environ.get("TP_TRANSPORT", "peer"))
    out_transport = tp.transport
    ref = ModelRunner(cfg, params=full, device=dev, num_blocks=64)
    shard = ModelRunner(cfg, params=InferenceWeights.shard_of(full, cfg, rank, world), device=dev, num_blocks=64, tp=tp)
    prompt = torch.randint(0, cfg.vocab_size, (77,), generator=torch.Generator().manual_seed(1)).tolist()
    out = {"world": world, "transport": out_transport}
    # go through the engines: same greedy tokens from both
    e_ref, e_tp = ServingEngine(ref), ServingEngine(shard)
    t_ref = e_ref.generate(prompt, 12)
    t_tp = e_tp.generate(prompt, 12)
    out["tokens_ref"], out["tokens_tp"] = t_ref, t_tp
    # logits of a fresh prefill
    e_ref2, e_tp2 = ServingEngine(ref), ServingEngine(shard)
    rid_a = e_ref2.scheduler.add_request(prompt, 4)
    rid_b = e_tp2.scheduler.add_request(prompt, 4)
    ba, bb = e_ref2.scheduler.schedule(), e_tp2.scheduler.schedule()
    la = ref.prefill(ba.request_ids[0], ba.input_ids[0]).float()
    lb = shard.prefill(bb.request_ids[0], bb.input_ids[0]).float()
    out["prefill_rel_err"] = float((la - lb).norm() / la.norm())
    # every rank must hold bit-identical logits
    gathered = [torch.empty_like(lb) for _ in range(world)]
    dist.all_gather(gathered, lb)
    out["ranks_identical"] = all(torch.equal(gathered[0], g) for g in gathered)
    torch.cuda.synchronize()
    st = torch.tensor([_native.read_status()[0]], device=dev)
    dist.all_reduce(st, op=dist.ReduceOp.MAX)
    out["status_max"] = int(st)
    dist.barrier()
    tp.close()
    if rank == 0:
        print(json.dumps(out))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
