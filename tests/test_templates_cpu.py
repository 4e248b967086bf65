"""Named chat templates: layout of the turns, supervised spans, media expansion, the no-think variant."""
from mindspeed_mm_b200.data.multimodal import ByteTokenizer
from mindspeed_mm_b200.data.templates import TEMPLATES, get_template


class _CharTok:
    """One id per character; special tokens get ids from 1000 on (whole-token match)."""
    eos_token, bos_token, unk_token_id = "</s>", "<s>", -1

    def __init__(self, specials):
        self.special_ids = {t: 1000 + i for i, t in enumerate(specials)}

    def encode(self, text, add_special_tokens=False):
        out, i = [], 0
        while i < len(text):
            for t, tid in self.special_ids.items():
                if text.startswith(t, i):
                    out.append(tid)
                    i += len(t)
                    break
            else:
                out.append(ord(text[i]))
                i += 1
        return out

    def decode(self, ids):
        inv = {v: k for k, v in self.special_ids.items()}
        return "".join(inv.get(i, chr(i)) if i < 1000 or i in inv else "?" for i in ids)


def test_registry_has_the_reference_names():
    for n in ("qwen2vl", "qwen3_vl", "qwen3_vl_nothink", "qwen2_omni", "qwen3_omni", "qwen3_omni_nothink", "glm4.1v", "glm4v_moe",
              "mistral", "default"):
        assert n in TEMPLATES


def test_qwen_layout_labels_and_media():
    tok = _CharTok(["<|im_start|>", "<|im_end|>", "<|vision_start|>", "<|vision_end|>", "<|image_pad|>", "<|video_pad|>"])
    t = get_template("qwen2vl", tok)
    ids, labels = t.render([{"role": "user", "content": "<image>what?"}, {"role": "assistant", "content": "a cat"}], [3], ["image"])
    text = tok.decode(ids)
    assert text == ("<|im_start|>system\nYou are a helpful assistant.<|im_end|>\n<|im_start|>user\n<|vision_start|><|image_pad|><|image_pad|>"
                    "<|image_pad|><|vision_end|>what?<|im_end|>\n<|im_start|>assistant\na cat<|im_end|>\n")
    sup = tok.decode([l for l in labels if l != -100])
    assert sup == "a cat<|im_end|>\n" and len(ids) == len(labels)
    nothink = get_template("qwen3_vl_nothink", tok).render([{"role": "user", "content": "hi"}, {"role": "assistant", "content": "yo"}])
    assert tok.decode([l for l in nothink[1] if l != -100]) == "<think>\n\n</think>\n\nyo<|im_end|>\n"


def test_glm_and_mistral_layouts():
    tok = _CharTok(["[gMASK]", "<sop>", "<|user|>", "<|assistant|>", "<|system|>", "<|begin_of_image|>", "<|end_of_image|>", "<|image|>"])
    ids, labels = get_template("glm4v_moe", tok).render(
        [{"role": "system", "content": "S"}, {"role": "user", "content": "<image>Q"}, {"role": "assistant", "content": "A"}], [2], ["image"])
    assert tok.decode(ids) == "[gMASK]<sop><|system|>\nS<|user|>\n<|begin_of_image|><|image|><|image|><|end_of_image|>Q<|assistant|>\nA"
    assert tok.decode([l for l in labels if l != -100]) == "\nA"                 # efficient eos: no end token after the answer
    tok2 = _CharTok(["[INST]", "[/INST]", "[IMG]", "[IMG_END]", "</s>", "<s>"])
    ids, labels = get_template("mistral", tok2).render([{"role": "user", "content": "<image>Q"}, {"role": "assistant", "content": "A"}], [2], ["image"])
    assert tok2.decode(ids) == "<s>[INST][IMG][IMG][IMG_END]Q[/INST]A</s>" and tok2.decode([l for l in labels if l != -100]) == "A</s>"


def test_marker_count_mismatch_is_an_error():
    tok = _CharTok(["<|im_start|>", "<|im_end|>", "<|vision_start|>", "<|vision_end|>", "<|image_pad|>", "<|video_pad|>"])
    t = get_template("qwen3_vl", tok)
    for msgs, counts in (([{"role": "user", "content": "<image><image>"}], [1]), ([{"role": "user", "content": "none"}], [1])):
        try:
            t.render(msgs, counts, ["image"] * len(counts))
            raise AssertionError
        except ValueError:
            pass
