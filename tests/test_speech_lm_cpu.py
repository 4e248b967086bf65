"""Speech-token LMs: delay pattern, channel losses, CosyVoice3 sequence layouts, Qwen3-TTS talker + code predictor."""
import torch

from mindspeed_mm_b200.models.speech_lm import (IGNORE, CosyVoice3Config, CosyVoice3LM, MultiCodebookConfig, MultiCodebookLM,
                                                Qwen3TTSConfig, Qwen3TTSTalker, SpeakerEncoder, apply_delay_pattern,
                                                label_smoothing_loss, ras_sampling, revert_delay_pattern)


def test_delay_pattern_roundtrip():
    codes = torch.arange(20).reshape(5, 4)
    d = apply_delay_pattern(codes, 99)
    assert d.shape == (8, 4) and d[0].tolist() == [0, 99, 99, 99] and d[-1].tolist() == [99, 99, 99, 19]
    assert torch.equal(revert_delay_pattern(d), codes)


def test_multicodebook_channel_losses_and_masked_pad_code():
    torch.manual_seed(0)
    m = MultiCodebookLM(MultiCodebookConfig.tiny(channel_loss_weight=[1.0, 2.0, 2.0, 2.0]))
    m.init_weights()
    T = 12
    ids = torch.randint(0, 30, (T, 4))
    lab = ids.roll(-1, 0).clone()
    lab[-1] = IGNORE
    lab[:, 3] = IGNORE                                    # a channel without labels contributes nothing
    b = dict(input_ids=ids, labels=lab, cu_seqlens=torch.tensor([0, 5, 12], dtype=torch.int32), max_seqlen=7)
    loss = m(b)
    cl = m.last_channel_losses
    assert float(cl[3]) == 0 and torch.allclose(loss, (cl[0] + 2 * cl[1] + 2 * cl[2]) / 7.0, atol=1e-5)
    loss.backward()
    assert m.emb_ext.weight.grad is not None and m.heads.extra[2].grad is None and float(m.heads.extra[0].grad.abs().sum()) > 0
    logits = m(dict(input_ids=ids, cu_seqlens=b["cu_seqlens"], max_seqlen=7))
    assert logits[0].shape == (T, 1024) and logits[1].shape == (T, 32)      # pad code (index 32) is not predicted
    names = [n for n, _ in m.fsdp_units()]
    assert "emb_ext" in names and "backbone.layers.0" in names and "heads" in names and "backbone.lm_head" not in names
    codes = m.eval().generate_codes(ids[:4], steps=3)
    assert codes.shape == (3, 3) and int(codes.max()) < 32


def test_cosyvoice3_layouts_loss_and_sampling():
    torch.manual_seed(0)
    c = CosyVoice3LM(CosyVoice3Config.tiny(lsm_weight=0.0))
    c.init_weights()
    S = c.config.speech_token_size
    kinds, ids, tgt = c.build_sample([1, 2, 3], [10, 11], instruct=[7, 8])
    assert ids == [S, 7, 8, 1, 2, 3, S + 2, 10, 11] and tgt == [IGNORE] * 6 + [10, 11, S + 1]
    assert "".join(kinds) == "s" + "t" * 5 + "sss"
    kinds, ids, tgt = c.build_sample([1, 2, 3, 4, 5], list(range(10, 27)), bistream=True)      # mix ratio 2 : 6
    assert ids[:9] == [S, 1, 2, 10, 11, 12, 13, 14, 15] and tgt[:9] == [IGNORE, IGNORE, 10, 11, 12, 13, 14, 15, S + 3]
    assert ids[-7:] == [5, S + 2, 22, 23, 24, 25, 26] and tgt[-6:] == [22, 23, 24, 25, 26, S + 1]
    # too little speech for the interleaved form: falls back to the sequential layout
    assert c.build_sample([1, 2, 3, 4], [10, 11], bistream=True) == c.build_sample([1, 2, 3, 4], [10, 11])
    batch = c.eval().pack([dict(text=[1, 2, 3], speech=[5, 6, 7, 8]), dict(text=[4, 5], speech=[9, 10, 11], instruct=[7])])
    assert batch["cu_seqlens"].tolist() == [0, 9, 17]
    loss = c(batch)
    loss.backward()
    assert c.speech_embedding.weight.grad is not None and c.heads.extra[0].grad is not None and c.backbone.lm_head.weight is None
    # label smoothing: equals plain CE at 0 smoothing
    logits, target = torch.randn(6, 11), torch.tensor([1, 2, IGNORE, 4, 5, 0])
    ce = torch.nn.functional.cross_entropy(logits, target, ignore_index=IGNORE)
    assert torch.allclose(label_smoothing_loss(logits, target, 0.0, True), ce, atol=1e-5)
    assert float(label_smoothing_loss(logits, target, 0.1, True)) > 0
    g = torch.Generator().manual_seed(0)
    scores = torch.full((50,), -10.0)
    scores[3] = 10.0
    assert ras_sampling(scores, [], generator=g) == 3
    mild = torch.zeros(50)
    mild[3] = 1.0
    picks = {ras_sampling(mild, [3] * 10, top_p=0.01, top_k=1, generator=g) for _ in range(20)}
    assert len(picks) > 1                                   # a repeated token triggers the redraw from the full distribution
    out = c.generate([1, 2, 3], max_len=4, min_len=4, generator=torch.Generator().manual_seed(0))
    assert len(out) == 4 and max(out) < S


def test_qwen3tts_talker_and_code_predictor():
    torch.manual_seed(0)
    cfg = Qwen3TTSConfig.tiny()
    m = Qwen3TTSTalker(cfg)
    m.init_weights()
    for p in m.speaker_front.encoder.parameters():
        torch.nn.init.normal_(p, std=0.05)
    G = cfg.num_code_groups
    s1 = m.build_sample([5, 6, 7], torch.randint(0, 60, (4, G)), bos=61, eos=62, pad=63)
    s2 = m.build_sample([8, 9], torch.randint(0, 60, (3, G)), bos=61, eos=62, pad=63)
    assert s1["length"] == 1 + 3 + 1 + 4 and s1["labels"].tolist()[:4] == [IGNORE] * 4
    assert s1["labels"][4:8].tolist() == s1["label_codec_ids"][:, 0].tolist() and int(s1["labels"][-1]) == 62
    assert s1["codec_in"][5:].tolist() == s1["label_codec_ids"][:, 0].tolist()      # teacher forcing: frame f feeds row f + 1
    batch = m.pack([s1, s2], ref_mels=torch.randn(2, 30, cfg.n_mels))
    assert batch["cu_seqlens"].tolist() == [0, 9, 16] and batch["speaker_pos"].tolist() == [0, 9] and batch["eos_rows"].tolist() == [8, 15]
    loss = m(batch)
    assert torch.isfinite(loss) and float(m.last_sub_talker_loss) > 0
    loss.backward()
    assert m.code_predictor.heads.weight.grad is not None and m.code_predictor.codec_embedding.weight.grad is not None
    assert m.text_front.fc1.weight.grad is not None
    assert all(p.grad is None for p in m.speaker_front.encoder.parameters()) and m.speaker_front.proj.weight.grad is not None            # speaker embedding is detached
    spk = SpeakerEncoder(20, 32, 16)(torch.randn(3, 25, 20))
    assert spk.shape == (3, 16)
    with torch.no_grad():
        hid = torch.randn(5, cfg.talker.hidden_size)
        code0 = torch.randint(0, 60, (5,))
        codes = m.code_predictor.generate(hid, code0, m.backbone.embed_tokens(code0))
    assert codes.shape == (5, G) and torch.equal(codes[:, 0], code0)
    names = [n for n, _ in m.fsdp_units()]
    assert "code_predictor.backbone.layers.0" in names and "backbone.layers.1" in names and "speaker_front" in names


def test_audio_codec_rvq_and_roundtrip_shapes():
    from mindspeed_mm_b200.models.audio_codec import (AudioCodec, AudioCodecConfig, CausalConv1d, ResidualVQ, VectorQuantize,
                                                      multi_scale_mel_loss)
    torch.manual_seed(0)
    # residual quantisation: every extra codebook lowers the reconstruction error
    rvq = ResidualVQ(4, 8, 64, ema_decay=None).eval()
    x = torch.randn(2, 8, 50)
    errs = [float((rvq(x, n)[0] - x).pow(2).mean()) for n in (1, 2, 4)]
    assert errs[0] > errs[1] > errs[2]
    codes = rvq.encode(x)
    assert codes.shape == (2, 4, 50) and torch.allclose(rvq.decode(codes), rvq(x)[0], atol=1e-5)
    # straight-through gradient and EMA update that moves the codebook toward the data
    vq = VectorQuantize(8, 16, ema_decay=0.5).train()
    xin = (torch.randn(2, 8, 40) * 3 + 5).requires_grad_()
    before = (vq.codebook.mean(0) - 5).abs().mean()
    q, idx, commit = vq(xin)
    q.sum().backward()
    assert torch.allclose(xin.grad, torch.ones_like(xin)) and idx.shape == (2, 40)
    assert (vq.codebook.mean(0) - 5).abs().mean() < before
    conv = CausalConv1d(1, 1, 5, stride=2)
    a = torch.randn(1, 1, 40)
    b = a.clone()
    b[..., 30:] += 1
    assert torch.equal(conv(a)[..., :15], conv(b)[..., :15])                     # output t depends on inputs <= 2t
    cfg = AudioCodecConfig.tiny()
    codec = AudioCodec(cfg)
    assert cfg.hop == 16
    wav = torch.randn(2, 1, 16 * 10 + 5)
    rec, codes, commit = codec(wav)
    assert rec.shape == wav.shape and codes.shape == (2, 4, 11) and torch.isfinite(commit)
    (multi_scale_mel_loss(rec, wav, 16000, ffts=(64, 128), n_mels=10) + commit).backward()
    assert codec.encoder[0].conv.weight.grad is not None and codec.decoder[-1].conv.weight.grad is not None
    codec.eval()
    c2 = codec.encode(wav)
    assert c2.shape == (2, 4, 11) and codec.decode(c2).shape[-1] >= wav.shape[-1]
