"""KL / VQ autoencoder family: wavelet identities, shape contracts, causal blocks, tiling, factory ids."""
import torch

from mindspeed_mm_b200.models.ae.kl_vae import (MOVQ, WFVAE, AutoencoderKL2D, CausalVAE3D, Conv, DiagonalGaussian, Down, KLVAEConfig,
                                                VectorQuantizer, _blend, haar, inverse_haar)
from mindspeed_mm_b200.models.towers import build_ae


def test_haar_is_orthonormal_and_low_band_first():
    torch.manual_seed(0)
    x = torch.randn(2, 3, 4, 8, 6)
    w = haar(x, (2, 3, 4))
    assert w.shape == (2, 24, 2, 4, 3)
    assert torch.allclose(inverse_haar(w, (2, 3, 4)), x, atol=1e-5)
    assert torch.allclose(w.pow(2).sum(), x.pow(2).sum(), rtol=1e-5)            # energy preserved
    blocks = x.reshape(2, 3, 2, 2, 4, 2, 3, 2).sum((3, 5, 7)) / (2 ** 1.5)
    assert torch.allclose(w[:, :3], blocks, atol=1e-5)
    w2 = haar(x, (3, 4))
    assert w2.shape == (2, 12, 4, 4, 3) and torch.allclose(inverse_haar(w2, (3, 4)), x, atol=1e-5)


def test_causal_conv_and_down_do_not_see_the_future():
    torch.manual_seed(0)
    conv, down = Conv(4, 4), Down(4, time=True)
    x = torch.randn(1, 4, 9, 8, 8)
    y = x.clone()
    y[:, :, 5:] += 1.0
    assert torch.equal(conv(x)[:, :, :5], conv(y)[:, :, :5])
    dx, dy = down(x), down(y)
    assert dx.shape == (1, 4, 5, 4, 4)
    assert torch.equal(dx[:, :, :3], dy[:, :, :3]) and not torch.equal(dx[:, :, 3:], dy[:, :, 3:])


def test_causal_vae_shapes_image_path_and_posterior():
    torch.manual_seed(0)
    v = CausalVAE3D(KLVAEConfig.tiny(scale_factor=0.5, shift_factor=0.1)).eval()
    assert v.compression() == (4, 4, 4)
    x = torch.randn(1, 3, 9, 16, 16)
    z = v.encode(x)
    assert z.shape == (1, 4, 3, 4, 4)
    assert v.decode(z).shape == x.shape
    img = torch.randn(2, 3, 16, 16)
    zi = v.encode(img)
    assert zi.shape == (2, 4, 4, 4) and v.decode(zi).shape == img.shape
    rec, post = v(x, sample_posterior=True, generator=torch.Generator().manual_seed(0))
    assert rec.shape == x.shape and post.kl().shape == (1,) and float(post.kl().detach()) >= 0
    g = DiagonalGaussian(torch.zeros(1, 8, 1, 2, 2))
    assert float(g.kl()) == 0 and torch.equal(g.mode(), torch.zeros(1, 4, 1, 2, 2))


def test_tiling_matches_shapes_and_blend_is_identity_on_constants():
    torch.manual_seed(0)
    a, b = torch.full((1, 1, 1, 4, 6), 2.0), torch.full((1, 1, 1, 4, 6), 2.0)
    assert torch.equal(_blend(a, b, 4, 3), b)
    ramp = _blend(torch.zeros(1, 1, 1, 1, 4), torch.ones(1, 1, 1, 1, 4), 4, 3)[0, 0, 0, 0]
    assert (ramp[1:] >= ramp[:-1]).all() and float(ramp[-1]) == 1 and 0 < float(ramp[0]) < 1
    v = CausalVAE3D(KLVAEConfig.tiny(), tile_sample_min=16, tile_overlap=0.25, tile_frames=5).eval()
    x = torch.randn(1, 3, 9, 32, 32)
    full = v.encode(x)
    v.enable_tiling()
    tiled = v.encode(x)
    assert tiled.shape == full.shape and torch.isfinite(tiled).all()
    out = v.decode(tiled)
    assert out.shape == x.shape and torch.isfinite(out).all()


def test_wfvae_and_movq_and_image_vae():
    torch.manual_seed(0)
    wf = WFVAE(base=16, z_channels=4, num_res_blocks=1, energy_flow=8).eval()
    x = torch.randn(1, 3, 9, 32, 32)
    z = wf.encode(x)
    assert z.shape == (1, 4, 3, 4, 4)
    rec, post = wf(x, sample_posterior=False)
    assert rec.shape == x.shape
    rec.mean().backward()
    assert wf.in_flow3[0].conv.weight.grad is not None and wf.out_flow2[1].conv.weight.grad is not None
    assert wf.get_last_layer().shape[0] == 24
    m = MOVQ(base=16, ch_mult=(1, 2, 2), num_res_blocks=1, n_embed=32).eval()
    img = torch.randn(2, 3, 16, 16)
    idx = m.encode(img)
    assert idx.shape == (2, 4, 4) and idx.dtype == torch.long and int(idx.max()) < 32
    assert m.decode_codes(idx).shape == img.shape
    vq = VectorQuantizer(8, 2)
    pts = vq.embedding.weight.detach()[[3, 5]].t().reshape(1, 2, 1, 2).clone().requires_grad_()
    ids, q, commit = vq(pts)
    assert ids.flatten().tolist() == [3, 5] and float(commit) < 1e-12
    q.sum().backward()
    assert torch.equal(pts.grad, torch.ones_like(pts))                              # straight-through
    k = AutoencoderKL2D(KLVAEConfig(base=16, ch_mult=(1, 2, 2, 2), num_res_blocks=1, kt=1, z_channels=4, scale_factor=0.36, shift_factor=0.1)).eval()
    zk = k.encode(img)
    assert zk.shape == (2, 4, 2, 2) and k.decode(zk).shape == img.shape
    assert sum(p.numel() for n, p in k.named_parameters() if "conv.weight" in n and p.shape[2] != 1) == 0   # no temporal taps


def test_factory_ids():
    tiny = dict(base=16, ch_mult=[1, 2, 2], num_res_blocks=1, z_channels=4)
    assert isinstance(build_ae(dict(model_id="casualvae", temporal_down=[True, True], **tiny)), CausalVAE3D)
    assert isinstance(build_ae(dict(model_id="autoencoder_kl_hunyuanvideo", temporal_down=[True, True], use_tiling=True, **tiny)), CausalVAE3D)
    assert isinstance(build_ae(dict(model_id="flux_vae", base=16, ch_mult=[1, 2, 2, 2], num_res_blocks=1)), AutoencoderKL2D)
    assert isinstance(build_ae(dict(model_id="vae", temporal_down=[False, False], **tiny)), AutoencoderKL2D)
    assert isinstance(build_ae(dict(model_id="wfvae", base=16, z_channels=4, num_res_blocks=1, energy_flow=8)), WFVAE)
    assert isinstance(build_ae(dict(model_id="movq", base=16, ch_mult=[1, 2, 2], num_res_blocks=1, n_embed=16)), MOVQ)


def test_ae_trainer_moving_average_follows_the_weights():
    import torch
    from mindspeed_mm_b200.runtime.ema import ModuleEMA
    lin = torch.nn.Linear(4, 4)
    ema = ModuleEMA(lin, decay=0.5)
    w0 = lin.weight.detach().clone()
    with torch.no_grad():
        lin.weight.add_(1.0)
    ema.update()
    assert torch.allclose(ema.shadow["weight"], w0 + 0.5)
    ema.apply_shadow()
    assert torch.allclose(lin.weight, w0 + 0.5)
    ema.restore()
    assert torch.allclose(lin.weight, w0 + 1.0)


def test_lpips_structure_loading_and_use_as_perceptual_term(tmp_path):
    import torch
    from mindspeed_mm_b200.models.ae.lpips import LPIPS, _CHANNELS
    from mindspeed_mm_b200.tasks.ae_train import VAELoss
    torch.manual_seed(0)
    net = LPIPS(use_dropout=True)
    # key layout of the published files: torchvision VGG-16 features + LPIPS linear heads
    assert getattr(net.net.slice3, "10").weight.shape == (256, 128, 3, 3) and net.lin4.model[1].weight.shape == (1, 512, 1, 1)
    assert all(not p.requires_grad for p in net.parameters())
    vgg = {}
    cin = 3
    for idxs, c in zip(((0, 2), (5, 7), (10, 12, 14), (17, 19, 21), (24, 26, 28)), _CHANNELS):
        for i in idxs:
            vgg[f"features.{i}.weight"], vgg[f"features.{i}.bias"] = torch.randn(c, cin, 3, 3) * 0.05, torch.zeros(c)
            cin = c
    vgg["classifier.0.weight"] = torch.zeros(4, 4)
    lin = {f"lin{i}.model.1.weight": torch.rand(1, c, 1, 1) for i, c in enumerate(_CHANNELS)}
    torch.save(vgg, tmp_path / "vgg16.pth")
    torch.save(lin, tmp_path / "vgg.pth")
    net = LPIPS(str(tmp_path / "vgg.pth"), str(tmp_path / "vgg16.pth"))
    assert torch.equal(getattr(net.net.slice4, "19").weight, vgg["features.19.weight"]) and torch.equal(net.lin2.model[1].weight, lin["lin2.model.1.weight"])
    x = torch.rand(2, 3, 32, 32) * 2 - 1
    y = (x + 0.3 * torch.randn_like(x)).clamp(-1, 1).requires_grad_()
    d0, d1 = net(x, x), net(x, y)
    assert d0.shape == (2,) and float(d0.abs().max()) == 0.0 and (d1 > 0).all()
    d1.sum().backward()
    assert y.grad is not None and float(y.grad.abs().sum()) > 0
    net.train()
    assert not net.training                                    # scoring stays deterministic
    v = torch.rand(1, 3, 2, 32, 32) * 2 - 1
    assert net(v, v.flip(2)).shape == (1,)
    loss = VAELoss(perceptual=net, perceptual_weight=0.5)
    out = loss.generator(x, y, torch.zeros(2, 4, 4, 4), torch.zeros(2, 4, 4, 4), step=0)
    assert torch.isfinite(out[0] if isinstance(out, tuple) else out).all()


def test_context_parallel_vae_matches_single_process():
    """Frames split over 3 gloo ranks (halo exchange for the causal convolutions, group-norm statistics over all ranks,
    first-frame handling of the temporal up-sampling on rank 0 only): moments, reconstruction, gradients."""
    import os
    import subprocess
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=3", "--master-addr", "127.0.0.1",
           "--master-port", str(29700 + os.getpid() % 200), os.path.join(here, "dist_cp_vae_check.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=dict(os.environ, OMP_NUM_THREADS="1"))
    assert r.returncode == 0 and "ok=True" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


def test_frame_counts_for_context_parallel_split():
    from mindspeed_mm_b200.parallel.cp.vae import frame_counts
    assert frame_counts(21, 2, 4) == [13, 8] and frame_counts(33, 4, 4) == [9, 8, 8, 8] and sum(frame_counts(49, 5, 4)) == 49
    import pytest
    with pytest.raises(ValueError):
        frame_counts(20, 2, 4)
    with pytest.raises(ValueError):
        frame_counts(5, 2, 4)
