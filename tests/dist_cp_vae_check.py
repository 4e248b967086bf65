"""Causal 3-D VAE with the frame axis split over the ranks (gloo): moments, reconstruction and parameter gradients equal
the single-process model on the whole clip."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mindspeed_mm_b200.models.ae.kl_vae import CausalVAE3D, KLVAEConfig  # noqa: E402
from mindspeed_mm_b200.parallel.cp import vae as cpv  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.manual_seed(0)
    cfg = KLVAEConfig.tiny()                                  # two temporal stride-2 stages: compression 4
    ref = CausalVAE3D(cfg).double()
    net = CausalVAE3D(cfg).double()
    net.load_state_dict(ref.state_dict())
    T = 1 + 4 * (2 * world + 1)                               # uneven split: some ranks get one block more
    x = torch.randn(1, 3, T, 16, 16, dtype=torch.double)

    mom = ref._moments(x)
    z = mom[:, : cfg.z_channels]
    rec = ref._decode(z)
    loss = rec.pow(2).sum() / rec.numel() + 1e-2 * mom.pow(2).sum()
    loss.backward()

    cpv.apply_context_parallel(net, dist.group.WORLD)
    counts = cpv.frame_counts(T, world, cfg.time_compression)
    xl = cpv.split_frames(x, dist.group.WORLD, cfg.time_compression)
    assert xl.shape[2] == counts[rank]
    mom_l = net._moments(xl)
    rec_l = net._decode(mom_l[:, : cfg.z_channels])
    lat_counts = [(c - (1 if r == 0 else 0)) // cfg.time_compression + (1 if r == 0 else 0) for r, c in enumerate(counts)]
    mom_all = cpv.gather_frames(mom_l.detach(), dist.group.WORLD, lat_counts)
    rec_all = cpv.gather_frames(rec_l.detach(), dist.group.WORLD, counts)
    ok = torch.allclose(mom_all, mom.detach(), atol=1e-9) and torch.allclose(rec_all, rec.detach(), atol=1e-9)
    if rank == 0 and os.environ.get("CP_VAE_DEBUG"):
        print("moments diff per frame", (mom_all - mom.detach()).abs().amax((0, 1, 3, 4)).tolist())
        print("recon diff per frame", (rec_all - rec.detach()).abs().amax((0, 1, 3, 4)).tolist())
    loss_l = rec_l.pow(2).sum() / rec.numel() + 1e-2 * mom_l.pow(2).sum()       # the ranks' terms add up to the full loss
    loss_l.backward()
    # a bias in front of a GroupNorm has a zero gradient up to rounding: errors are measured against the largest gradient
    scale = max(float(q.grad.abs().max()) for q in ref.parameters())
    worst = 0.0
    for (n, p), (_, q) in zip(net.named_parameters(), ref.named_parameters()):
        g = p.grad.clone()
        dist.all_reduce(g)
        worst = max(worst, float((g - q.grad).abs().max()) / scale)
    ok = ok and worst < 1e-9
    names_same = [n for n, _ in net.named_parameters()] == [n for n, _ in ref.named_parameters()]
    t = torch.tensor([float(ok and names_same)])
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(f"world={world} frames={counts} worst_grad_rel={worst:.2e} ok={bool(t.item())}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
