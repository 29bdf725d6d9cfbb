"""Run under torchrun: the NVLink uint8 all-reduce and the fused outer step against exact fp32 math."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from prime_b200.compression import uniform_8bit_quantize  # noqa: E402
from prime_b200.config import Compression  # noqa: E402
from prime_b200.ops.kernels import check_status  # noqa: E402
from prime_b200.parallel.diloco_comm import NvlinkWorkerGroup  # noqa: E402
from prime_b200.parallel.symm import SymmComm  # noqa: E402


class _FakeModel:
    def __init__(self, master):
        self.master = master


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    grp = NvlinkWorkerGroup(SymmComm(), 3_000_000)
    ok = True
    for n in (1000, 1 << 20, 2_500_003):
        torch.manual_seed(100 + rank)
        x = torch.randn(n, device="cuda") * 1e-3
        exact = x.clone()
        dist.all_reduce(exact)
        got = x.clone()
        grp.all_reduce_tensor(got, Compression.UINT8)
        err = ((got - exact).norm() / exact.norm()).item()
        # oracle: what one quantise -> dequantise of the exact sum would cost
        q, lut = uniform_8bit_quantize(exact.cpu())
        ref_err = ((lut[q.long()] - exact.cpu()).norm() / exact.cpu().norm()).item()
        chk = [torch.zeros(1, device="cuda", dtype=torch.float64) for _ in range(world)]
        dist.all_gather(chk, got.double().sum().reshape(1))
        same = all(float(c) == float(chk[0]) for c in chk)
        if n >= 1000 and (err > 3 * ref_err * (world ** 0.5) + 1e-3 or not same):
            print(f"[rank {rank}] n={n}: rel err {err:.4f} (single quantisation {ref_err:.4f}), identical={same}")
            ok = False
        if rank == 0:
            print(f"n={n}: uint8 all-reduce rel err {err:.4f}; single-quantisation floor {ref_err:.4f}; ranks identical: {same}")
    # fused outer step vs torch SGD(nesterov) fed with the exact mean pseudo-gradient
    n = 1_500_000
    torch.manual_seed(7)
    outer0 = torch.randn(n)
    torch.manual_seed(50 + rank)
    inner = (outer0 + 1e-3 * torch.randn(n)).cuda()
    outer_h, mom_h = outer0.clone().pin_memory(), torch.zeros(n).pin_memory()
    pg = (outer0.cuda() - inner)
    dist.all_reduce(pg)
    pg /= world
    ref_p = torch.nn.Parameter(outer0.clone())
    opt = torch.optim.SGD([ref_p], lr=0.7, momentum=0.9, nesterov=True)
    ref_p.grad = pg.cpu()
    opt.step()
    model = _FakeModel(inner)
    grp.fused_outer_step(model, outer_h, mom_h, lr=0.7, momentum=0.9, fake=False, compression=Compression.UINT8)
    upd_ref = ref_p.data - outer0
    upd_got = outer_h - outer0
    rel = ((upd_got - upd_ref).norm() / upd_ref.norm()).item()
    if rel > 0.08 or not torch.equal(model.master.cpu(), outer_h):
        print(f"[rank {rank}] fused outer step: update rel err {rel:.4f}, inner==outer {torch.equal(model.master.cpu(), outer_h)}")
        ok = False
    # second step with a fake (zero) contribution from the last rank
    model.master.add_(1e-3 * torch.randn(n, device="cuda"))
    grp.fused_outer_step(model, outer_h, mom_h, lr=0.7, momentum=0.9, fake=(rank == world - 1), compression=Compression.UINT8)
    check_status()
    # outer state resident on the device: two steps give the same outer parameters, momentum and inner shard, bit for
    # bit, as two steps that stage through the host; the host mirrors are valid after wait_host_copies(); a host copy
    # that was rewritten between steps (checkpoint load) is read again when the caller says so
    def two_steps(resident):
        torch.manual_seed(900 + rank)
        m = _FakeModel((outer0 + 1e-3 * torch.randn(n)).cuda())
        oh, mh = outer0.clone().pin_memory(), torch.zeros(n).pin_memory()
        grp._outer_dev = None                                   # start from the host copies
        for s_ in range(2):
            grp.fused_outer_step(m, oh, mh, lr=0.7, momentum=0.9, fake=False, compression=Compression.UINT8,
                                 resident=resident, host_changed=(s_ == 0))
            m.master.add_(1e-3 * torch.randn(n, device="cuda"))
        grp.wait_host_copies()
        return oh.clone(), mh.clone(), m, oh, mh
    o_st, m_st, _, _, _ = two_steps(False)
    o_re, m_re, mdl, oh, mh = two_steps(True)
    if not (torch.equal(o_st, o_re) and torch.equal(m_st, m_re)):
        print(f"[rank {rank}] resident outer state differs from the staged one")
        ok = False
    oh.copy_(outer0)                                            # the host copies are rewritten (as a checkpoint load does)
    mh.zero_()
    mdl.master.copy_((outer0 + 1e-3 * (1 + 0.1 * torch.randn(n))).cuda())
    grp.fused_outer_step(mdl, oh, mh, lr=0.7, momentum=0.9, fake=False, compression=Compression.UINT8, resident=True, host_changed=True)
    grp.wait_host_copies()
    want = -0.7 * 1.9 * 1e-3                                     # first Nesterov step from zero momentum: -lr * (1 + mu) * g, g = -1e-3
    if abs((oh - outer0).mean().item() + want) > 2e-4:
        print(f"[rank {rank}] rewritten host copies were not read again: mean update {(oh - outer0).mean().item():.6f}")
        ok = False
    check_status()
    # elastic membership, driven from the host between calls: the last rank leaves (it is not part of the next reduction),
    # then rejoins contributing a zero pseudo-gradient once
    torch.manual_seed(300 + rank)
    x = torch.randn(200_003, device="cuda") * 1e-3
    for members, fake_rank in ((list(range(world - 1)) or [0], None), (list(range(world)), world - 1)):
        grp.set_participants(members)
        contrib = x.clone()
        if rank not in members or rank == fake_rank:
            contrib.zero_()
        exact = contrib.clone()
        dist.all_reduce(exact)
        got = x.clone()
        grp.all_reduce_tensor(got, Compression.UINT8, fake=(rank == fake_rank))
        if rank in members:
            err = ((got - exact).norm() / exact.norm()).item()
            if err > 0.06:
                print(f"[rank {rank}] members {members} fake {fake_rank}: rel err {err:.4f}")
                ok = False
        elif not torch.equal(got, x):
            print(f"[rank {rank}] a rank outside the reduction had its tensor changed")
            ok = False
        assert grp.size() == len(members)
    grp.set_participants(list(range(world)))
    check_status()
    flag = torch.tensor([0 if ok else 1], device="cuda")
    dist.all_reduce(flag)
    if rank == 0:
        print(f"fused outer step update rel err {rel:.4f}")
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(1 if flag.item() else 0)


if __name__ == "__main__":
    main()
