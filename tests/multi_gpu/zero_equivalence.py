"""Run under torchrun with W ranks: the W-rank ZeRO engine on a split batch must match a 1-rank engine
on the whole batch (same weights, same data) — parameters after two optimizer steps, gradient norm
and loss. Exits non-zero on mismatch. ``--reshard`` runs the mode without a resident replica (blocks re-gathered when they
run, QKV gather fused into its GEMM), ``--ac`` adds activation checkpointing."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from prime_b200.engine.fused_llama import FusedLlama  # noqa: E402
from prime_b200.models.llama import ModelArgs, Transformer  # noqa: E402
from prime_b200.ops.kernels import check_status  # noqa: E402
from prime_b200.parallel.symm import SymmComm  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    args = ModelArgs(dim=256, n_layers=2, n_heads=4, n_kv_heads=2, ffn_hidden=768, vocab_size=1000, max_seq_len=256,
                     init_mode="normal", init_std=0.05)
    torch.manual_seed(0)
    model = Transformer(args)
    g = torch.Generator().manual_seed(1)
    B, T = 4 * world, 256
    tok = torch.randint(0, args.vocab_size, (2, B, T + 1), generator=g)
    reshard, ac = "--reshard" in sys.argv, "--ac" in sys.argv
    sharded = FusedLlama(args, device="cuda", comm=SymmComm(), ce_chunk_tokens=512, reshard=reshard, ac_ckpt=ac)
    sharded.load_from_module(model)
    single = FusedLlama(args, device="cuda", ce_chunk_tokens=512)
    single.load_from_module(model)
    per = B // world
    ok = True
    for step in range(2):
        x, y = tok[step, :, :-1].contiguous(), tok[step, :, 1:].contiguous()
        l1, n1 = single.train_step(x, y, lr=1e-3, micro_bs=per)          # accumulation over `world` micro-batches
        lw, nw = sharded.train_step(x[rank * per:(rank + 1) * per], y[rank * per:(rank + 1) * per], lr=1e-3, micro_bs=per)
        lt = torch.tensor([lw], device="cuda")
        dist.all_reduce(lt)
        lw_mean = lt.item() / world
        if abs(lw_mean - l1) > 2e-2 or abs(nw - n1) / n1 > 3e-2:
            print(f"[rank {rank}] step {step}: loss {lw_mean} vs {l1}, norm {nw} vs {n1}")
            ok = False
    check_status()
    # compare this rank's master shard with the same rows of the single-rank engine
    worst = 0.0
    for name, shard in sharded.named_master_shards():
        seg = sharded.layout.segments[rank][sharded.layout.by_name[name]]
        ref = dict(single.named_master_shards())[name][seg.row_start: seg.row_end]
        if shard.numel():
            worst = max(worst, ((shard - ref).norm() / (ref.norm() + 1e-12)).item())
    # and the bf16 replicas of all ranks must be bit-identical
    same = True
    if not reshard:
        mine = sharded.params.view(torch.int16).to(torch.int64).sum()
        allsum = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(allsum, mine)
        same = all(int(a) == int(allsum[0]) for a in allsum)
    if worst > 5e-3 or not same:
        print(f"[rank {rank}] shard mismatch {worst}, replicas identical: {same}")
        ok = False
    flag = torch.tensor([0 if ok else 1], device="cuda")
    dist.all_reduce(flag)
    dist.barrier()
    dist.destroy_process_group()
    if flag.item():
        sys.exit(1)
    if rank == 0:
        print(f"zero equivalence ok (reshard={reshard}, ac={ac}): worst shard rel err {worst:.2e}, "
              f"max memory {torch.cuda.max_memory_allocated() / 2 ** 20:.0f} MiB")


if __name__ == "__main__":
    main()
