"""Frozen towers (text / vision / audio encoders, video VAE): parity with transformers where a counterpart exists,
structural invariants (causality, chunked == one-shot) for the VAE."""
import torch

from mindspeed_mm_b200.models.ae.wan_vae import WanVAE, WanVAEConfig
from mindspeed_mm_b200.models.encoders import (CLIPVisionConfig, CLIPVisionEncoder, WhisperConfig, WhisperEncoder,
                                               WindowedAudioEncoder)
from mindspeed_mm_b200.models.text_encoder import CLIPTextConfig, CLIPTextEncoder, T5Config, T5Encoder, TextEncoder


def test_umt5_encoder_matches_transformers():
    from transformers import UMT5Config, UMT5EncoderModel
    torch.manual_seed(0)
    hc = UMT5Config(vocab_size=128, d_model=64, d_kv=16, d_ff=128, num_layers=2, num_heads=4,
                    relative_attention_num_buckets=32, relative_attention_max_distance=128,
                    feed_forward_proj="gated-gelu", dropout_rate=0.0)
    hf = UMT5EncoderModel(hc).eval()
    me = T5Encoder(T5Config.tiny()).eval()
    me.load_hf_state_dict(hf.state_dict())
    ids = torch.randint(0, 128, (2, 11))
    mask = torch.ones(2, 11, dtype=torch.long)
    mask[1, 7:] = 0
    with torch.no_grad():
        want = hf(input_ids=ids, attention_mask=mask).last_hidden_state
        got = me(ids, mask)
        enc = TextEncoder(me).encode(ids, mask)
    assert torch.allclose(got[mask.bool()], want[mask.bool()], atol=1e-5)
    assert enc[1, 7:].abs().max() == 0


def test_clip_text_and_vision_match_transformers():
    from transformers import CLIPTextConfig as HT, CLIPTextModel, CLIPVisionConfig as HV, CLIPVisionModel
    torch.manual_seed(0)
    hf = CLIPTextModel(HT(vocab_size=100, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                          num_attention_heads=4, max_position_embeddings=16, eos_token_id=99, bos_token_id=0,
                          pad_token_id=1)).eval()
    me = CLIPTextEncoder(CLIPTextConfig.tiny()).eval()
    me.load_hf_state_dict(hf.state_dict())
    ids = torch.randint(2, 98, (2, 9))
    ids[:, -1] = 99
    with torch.no_grad():
        o = hf(input_ids=ids)
        h, p = me(ids)
    assert torch.allclose(h, o.last_hidden_state, atol=1e-5) and torch.allclose(p, o.pooler_output, atol=1e-5)

    hf = CLIPVisionModel(HV(image_size=28, patch_size=14, hidden_size=64, intermediate_size=128, num_hidden_layers=3,
                            num_attention_heads=4)).eval()
    me = CLIPVisionEncoder(CLIPVisionConfig.tiny()).eval()
    me.load_hf_state_dict(hf.state_dict())
    px = torch.randn(2, 3, 28, 28)
    with torch.no_grad():
        o = hf(pixel_values=px, output_hidden_states=True)
        h, p = me(px)
        pen = me.encode(px)
    assert torch.allclose(h, o.last_hidden_state, atol=1e-5) and torch.allclose(p, o.pooler_output, atol=1e-5)
    assert torch.allclose(pen, o.hidden_states[-2], atol=1e-5)


def test_whisper_encoder_matches_transformers_and_windowed_tower_shapes():
    from transformers import WhisperConfig as HW
    from transformers.models.whisper.modeling_whisper import WhisperEncoder as HWE
    torch.manual_seed(0)
    hf = HWE(HW(num_mel_bins=16, d_model=64, encoder_ffn_dim=128, encoder_layers=2, encoder_attention_heads=4,
                max_source_positions=50)).eval()
    me = WhisperEncoder(WhisperConfig.tiny()).eval()
    me.load_hf_state_dict(hf.state_dict(), prefix="")
    mel = torch.randn(2, 16, 100)
    with torch.no_grad():
        assert torch.allclose(me(mel), hf(mel).last_hidden_state, atol=1e-5)
        tower = WindowedAudioEncoder(WhisperConfig.tiny(), n_window=20, output_dim=32).eval()
        a, b = tower([torch.randn(16, 90), torch.randn(16, 37)])
    assert a.shape == (22, 32) and b.shape == (9, 32)


def test_wan_vae_causal_and_chunked_equals_one_shot():
    torch.manual_seed(0)
    vae = WanVAE(WanVAEConfig.tiny()).eval()
    for p in vae.parameters():
        p.data.normal_(0, 0.2)
    video = torch.rand(1, 3, 13, 32, 32) * 2 - 1
    z = vae.encode(video)
    assert z.shape == (1, 4, 4, 4, 4) and vae.compression == (4, 8, 8)
    assert torch.allclose(vae.encode(video[:, :, :5]), z[:, :, :2], atol=1e-6)          # causal in time
    assert torch.allclose(vae.encode(video, chunk_frames=4), z, atol=1e-5)
    x = vae.decode(z)
    assert x.shape == video.shape
    assert torch.allclose(vae.decode(z, chunk_frames=1), x, atol=1e-4)


def test_wan_vae_full_size_parameter_count():
    n = sum(p.numel() for p in WanVAE().parameters())
    assert 126e6 < n < 128e6
