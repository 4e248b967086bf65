"""Prompt encoders of the HunyuanVideo family: template cropping, inner-layer read-out, glyph byte encoder."""
import torch

from mindspeed_mm_b200.models import prompt_encoders as pe


def _encode(s):
    return [3 + (ord(c) % 500) for c in s]


def test_templates_and_crop_measurement():
    t = pe.TEMPLATES["encode-video"]
    text = pe.apply_template("a cat", t["template"])
    assert text.endswith("a cat<|eot_id|>")
    chat = pe.apply_template("", pe.TEMPLATES["encode-video-chat"]["template"])
    assert chat[1]["content"] == " " and pe.TEMPLATES["encode-video-chat"]["template"][1]["content"] == "{}"
    crop = pe.measure_crop_start(t["template"], _encode)
    assert crop == len(t["template"].split("{}")[0])
    tpl = pe.resolve_template(pe.TEMPLATES["encode-video-chat"], _encode)
    ids, mask = pe.tokenize_prompts(["hello", "a much longer prompt"], _encode, tpl, max_length=8)
    assert ids.shape == (2, 8 + tpl["crop_start"]) and mask[:, : tpl["crop_start"]].all()
    # the first prompt token sits right after the cropped prefix
    assert ids[0, tpl["crop_start"]] == _encode("h")[0] and ids[1, tpl["crop_start"]] == _encode("a")[0]


def test_decoder_prompt_encoder_reads_an_inner_layer_and_crops():
    from mindspeed_mm_b200.models.composable import PRESETS, ComposableLM
    from dataclasses import replace
    cfg = PRESETS["llava"]
    cfg = replace(cfg, text=replace(cfg.text, num_layers=3, mixers=(), ffns=()), vision_kind=None)
    torch.manual_seed(0)
    lm = ComposableLM(cfg)
    with torch.no_grad():
        lm.init_weights(0)
    tpl = {"template": "SYS: {}", "crop_start": 5}
    enc = pe.DecoderPromptEncoder(lm, tpl, skip_layer=2)
    ids, mask = pe.tokenize_prompts(["ab", "abcdef"], lambda s: [1 + ord(c) % 100 for c in s], tpl, max_length=6)
    h, m = enc.encode(ids, mask)
    assert h.shape == (2, 6, cfg.text.hidden_size) and m.shape == (2, 6)
    assert m.sum(1).tolist() == [2, 6]
    # skip_layer counts from the last layer: 2 -> output of layer 1 of 3
    T = int(mask[1].sum())
    batch = dict(input_ids=ids[1, :T], position_ids=torch.arange(T), cu_seqlens=torch.tensor([0, T], dtype=torch.int32), max_seqlen=T)
    hs = lm.hidden_states(batch)
    assert len(hs) == 4
    assert torch.allclose(h[1, : T - 5], hs[1][5:], atol=1e-5)
    assert float(h[0, 2:].abs().max()) == 0.0                       # padded positions stay zero
    # causal LM: another sample in the batch does not change a sample's states
    h_alone, _ = enc.encode(ids[1:], mask[1:])
    assert torch.allclose(h_alone[0], h[1], atol=1e-5)
    last = pe.DecoderPromptEncoder(lm, tpl, skip_layer=0).encode(ids, mask)[0]
    assert torch.allclose(last[1, : T - 5], hs[-1][5:], atol=1e-5)


def test_glyph_extraction_formatting_and_byte_tokenizer():
    assert pe.extract_glyph_texts('A sign says "OPEN" and “欢迎” and "OPEN" again') == ["OPEN", "欢迎"]
    assert pe.extract_glyph_texts('no quotes, or an "unclosed one') == []
    assert pe.format_glyph_prompt(["OPEN", "hi"]) == 'Text "OPEN". Text "hi". '
    colors, fonts = {"red": 0, "blue": 1}, {"en-Arial": 0, "cn-Song": 1}
    s = pe.format_glyph_prompt(["A"], [{"color": "blue", "font-family": "cn-Song"}], colors, fonts)
    assert s == 'Text "A" in <color-1>, <cn-font-1>. '
    tok = pe.ByteTokenizer.with_styles(colors, fonts)
    assert len(tok) == 384 + 4
    ids = tok.encode(s)
    assert ids[-1] == tok.eos_id and 384 + 1 in ids and 384 + 2 + 1 in ids
    assert tok.decode(ids) == s
    assert tok.encode("é", add_eos=False) == [0xC3 + 3, 0xA9 + 3]
    i, m = tok("abc", 6)
    assert i.tolist() == [[100, 101, 102, 1, 0, 0]] and m.tolist() == [[1, 1, 1, 1, 0, 0]]


def test_glyph_encoder_zero_for_prompts_without_quotes():
    from mindspeed_mm_b200.models.registry import build_model
    torch.manual_seed(0)
    enc = build_model("hunyuan15_glyph_encoder", {"preset": "tiny"})
    for p in enc.parameters():
        torch.nn.init.normal_(p, std=0.05)
    emb, mask = enc.encode_prompts(['a shop sign that reads "OPEN"', "a quiet street"])
    assert emb.shape == (2, 24, 32) and mask.shape == (2, 24)
    assert mask[0].sum() == len('Text "OPEN". ') + 1 and mask[1].sum() == 0
    assert float(emb[1].abs().max()) == 0.0 and float(emb[0].abs().max()) > 0
    assert all(not p.requires_grad for p in enc.parameters())
    full = pe.GlyphEncoderConfig()
    assert (full.d_model, full.vocab_size, full.max_length) == (1472, 1510, 256)


def test_text_encoder_builder_knows_both_branches():
    from mindspeed_mm_b200.models.towers import build_text_encoder
    te = build_text_encoder([{"model_id": "hunyuan15_mllm", "lm_model_id": "llava", "template": {"template": "S {}", "crop_start": 2}},
                             {"model_id": "hunyuan15_glyph_byt5", "preset": "tiny"}])
    ids = [torch.randint(3, 100, (2, 10)), torch.randint(3, 100, (2, 24))]
    (h, m), (g, gm) = te.encode(ids, [torch.ones(2, 10, dtype=torch.long), torch.ones(2, 24, dtype=torch.long)])
    assert h.shape == (2, 8, 128) and m.shape == (2, 8) and g.shape == (2, 24, 32) and gm.shape == (2, 24)


def test_stepllm_encoder_bias_and_causality():
    s = pe.alibi_slopes(8)
    assert torch.allclose(s, torch.tensor([2.0 ** -(i + 1) for i in range(8)]))
    s6 = pe.alibi_slopes(6)                                          # 4 from the power-of-two series, 2 interleaved
    assert s6.shape == (6,) and torch.allclose(s6[:4], torch.tensor([0.25, 0.0625, 0.015625, 0.00390625]))
    assert torch.allclose(s6[4:], torch.tensor([0.5, 0.125]))
    b = pe.sqrt_alibi_bias(5, 2)
    assert b.shape == (2, 5, 5) and b[0, 0, 1] == float("-inf") and b[0, 2, 2] == 0
    assert abs(float(b[0, 4, 0]) + float(pe.alibi_slopes(2)[0]) * 2.0) < 1e-6      # sqrt(4) = 2
    from mindspeed_mm_b200.models.registry import build_model
    torch.manual_seed(0)
    m = build_model("stepllm", {"preset": "tiny"})
    for p in m.parameters():
        if p.dim() > 1:
            torch.nn.init.normal_(p, std=0.1)
    ids = torch.randint(0, 128, (2, 9))
    h, mask = m.encode(ids)
    assert h.shape == (2, 9, 96) and mask.shape == (2, 9)
    ids2 = ids.clone()
    ids2[:, 6:] = (ids2[:, 6:] + 1) % 128
    h2, _ = m.encode(ids2)
    assert torch.allclose(h[:, :6], h2[:, :6], atol=1e-6) and not torch.allclose(h[:, 6:], h2[:, 6:])
    # without positions in the embeddings, order still matters through the bias
    perm = torch.tensor([1, 0, 2, 3, 4, 5, 6, 7, 8])
    assert not torch.allclose(m.encode(ids[:, perm])[0][:, 8], h[:, 8], atol=1e-5)
    # feed-forward width is rounded up to the configured multiple
    assert m.layers[0].w2.in_features == 112 and m.layers[0].wqkv.out_features == 96 + 2 * 16 * 2
