"""Image-to-video conditioning builders against a toy VAE (8x spatial, 4x temporal average pooling)."""
import torch
import torch.nn.functional as F

from mindspeed_mm_b200.tasks import i2v_processors as ip


class ToyVAE:
    scaling_factor = 0.5

    def encode(self, x):                       # [B, 3, T, H, W] -> [B, 4, 1 + (T-1)/4, H/8, W/8]
        first = F.avg_pool3d(x[:, :, :1], (1, 8, 8))
        rest = F.avg_pool3d(x[:, :, 1:], (4, 8, 8)) if x.shape[2] > 1 else x[:, :, :0, ::8, ::8]
        lat = torch.cat([first, rest], 2)
        return torch.cat([lat, lat[:, :1]], 1) * self.scaling_factor

    def decode(self, z):                       # [B, 4, t, h, w] -> [B, 3, t, 8h, 8w]
        return F.interpolate(z[:, :3], scale_factor=(1, 8, 8), mode="nearest")


def _inputs():
    torch.manual_seed(0)
    vae = ToyVAE()
    videos = torch.rand(2, 3, 9, 16, 32) * 2 - 1
    return vae, videos, vae.encode(videos)


def test_cogvideox_and_stepvideo_first_frame_latents():
    vae, videos, lat = _inputs()
    out = ip.CogVideoXI2V({"noised_image_dropout": 0.0, "noised_image_input": False})(vae, videos, lat)["masked_video"]
    assert out.shape == lat.shape and torch.allclose(out[:, :, 0], lat[:, :, 0]) and float(out[:, :, 1:].abs().max()) == 0
    noisy = ip.CogVideoXI2V({"noised_image_dropout": 0.0}, seed=1)(vae, videos, lat)["masked_video"]
    d = (noisy[:, :, 0] - lat[:, :, 0]).abs().max()
    assert 0 < d < 0.2                                           # sigma = exp(N(-3, 0.5)) ~ 0.05, averaged over 8 x 8 pixels
    rep = ip.CogVideoXI2V({"noised_image_dropout": 0.0, "noised_image_input": False, "noised_image_all_concat": True})(vae, videos, lat)
    assert torch.allclose(rep["masked_video"][:, :, 2], lat[:, :, 0])
    dropped = ip.CogVideoXI2V({"noised_image_dropout": 1.0})(vae, videos, lat)["masked_video"]
    assert float(dropped.abs().max()) == 0
    st = ip.StepVideoI2V(seed=2)(vae, videos, lat)["image_latents"]
    assert st.shape == lat.shape and float(st[:, :, 1:].abs().max()) == 0 and float(st[:, :, 0].abs().max()) > 0
    a = ip.add_lognormal_noise(torch.zeros(4000, 1), torch.Generator().manual_seed(0))
    assert 0.03 < float(a.abs().median()) / 0.6745 < 0.08        # median |N(0, sigma)| = 0.6745 sigma, sigma ~ e^-3


def test_opensoraplan_mask_folding():
    vae, videos, lat = _inputs()
    mask = torch.zeros(2, 1, 9, 16, 32)
    mask[:, :, 1:] = 1                                            # frame 0 is given, the rest is to be generated
    mask[:, :, 0, :8, :8] = 1                                      # ... except one block of frame 0
    m = ip.compress_mask(mask, 4, 8, 8)
    assert m.shape == (2, 4 * 8 * 8, 3, 2, 4)
    assert float(m[:, :, 0, 0, 0].min()) == 1 and float(m[:, :, 0, 1, 1].max()) == 0 and float(m[:, :, 1:].min()) == 1
    proc = ip.build_i2v_processor({"processor_id": "opensoraplan_i2v_processor"})
    out = proc(vae, videos, lat, masked_video=videos * (1 - mask), input_mask=mask)
    assert out["masked_video"].shape == lat.shape and out["input_mask"].shape == m.shape
    try:
        proc(vae, videos, lat)
        raise AssertionError("missing mask must be reported")
    except ValueError:
        pass


def test_hunyuan_processors():
    vae, videos, lat = _inputs()
    out = ip.HunyuanVideoI2V({"image_size": 24}, seed=0)(vae, videos, lat)
    assert out["cond_latents"].shape == (2, 4, 1, 2, 4) and out["pixel_value_llava"].shape == (2, 3, 24, 24)
    assert int(out["uncond"]) == 0
    black = ip.HunyuanVideoI2V({"image_size": 24, "sematic_cond_drop_p": 1.0}, seed=0)(vae, videos, lat)
    assert int(black["uncond"]) == 1 and not torch.allclose(black["pixel_value_llava"], out["pixel_value_llava"])
    assert torch.allclose(black["cond_latents"], out["cond_latents"])          # only the semantic branch is dropped
    o15 = ip.HunyuanVideo15I2V(vision_tower=lambda img: img.flatten(2).transpose(1, 2)[:, :5])(vae, videos, lat)
    c = o15["cond_latents"]
    assert c.shape == (2, 5, 3, 2, 4) and torch.equal(c[:, :4, 0], lat[:, :, 0]) and float(c[:, 4, 0].min()) == 1
    assert float(c[:, :, 1:].abs().max()) == 0 and o15["vision_states"].shape == (2, 5, 3)
    assert "vision_states" not in ip.HunyuanVideo15I2V()(vae, videos, lat)
    assert ip.build_i2v_processor(None) is None
    try:
        ip.build_i2v_processor({"processor_id": "nope"})
        raise AssertionError
    except ValueError:
        pass
