"""Benchmark tables -> prompts -> scores."""
import base64
import io

from mindspeed_mm_b200.tasks import eval_datasets as ed
from mindspeed_mm_b200.tasks.evaluation import evaluate


def _png():
    from PIL import Image
    buf = io.BytesIO()
    Image.new("RGB", (4, 4), (255, 0, 0)).save(buf, format="PNG")
    return base64.b64encode(buf.getvalue()).decode()


def _write(path, header, rows):
    with open(path, "w", encoding="utf-8") as f:
        f.write("\t".join(header) + "\n")
        for r in rows:
            f.write("\t".join(r) + "\n")


def test_mmmu_prompt_places_pictures_at_their_tags(tmp_path):
    img = _png()
    p = tmp_path / "mmmu.tsv"
    _write(p, ["index", "question", "A", "B", "C", "hint", "answer", "category", "image"],
           [["1", "Compare <image 1> with <image 2>.", "same", "different", "", "look closely", "B", "Art", f"['{img}', '{img}']"],
            ["2", "What colour?", "red", "blue", "green", "", "A", "Design", "1"]])
    ds = ed.build_eval_dataset("MMMU_DEV_VAL", str(p))
    s = list(ds.samples())
    kinds = [m["type"] for m in s[0]["messages"]]
    assert kinds == ["text", "image", "text", "image", "text"]
    assert s[0]["messages"][0]["value"] == "Hint: look closely\nQuestion: Compare "
    assert s[0]["messages"][-1]["value"].startswith(".\nOptions:\nA. same\nB. different\nPlease select")
    assert "C." not in s[0]["messages"][-1]["value"]
    # row 2 borrows the pictures of row 1 and has no tag: pictures first
    assert [m["type"] for m in s[1]["messages"]] == ["image", "image", "text"] and s[1]["messages"][0]["value"].size == (4, 4)
    res = evaluate(lambda smp: "B" if smp["index"] == "1" else "The answer is (C)", ds.samples(), "multiple_choice")
    assert res["accuracy"] == 0.5 and res["per_category"] == {"Art": 1.0, "Design": 0.0}
    ds.write_predictions({"1": "B", "2": "C"}, str(tmp_path / "out.tsv"))
    out = ed.read_table(str(tmp_path / "out.tsv"))
    assert out[1]["prediction"] == "C" and "image" not in out[0]
    assert sum(1 for _ in ds.samples(1, 2)) == 1
    try:
        ed.split_at_image_tags("see <image x>", [])
        raise AssertionError
    except ValueError:
        pass


def test_vqa_dataset_and_anls(tmp_path):
    p = tmp_path / "doc.tsv"
    _write(p, ["index", "question", "answer", "image"], [["7", "Total?", "['42', 'forty two']", _png()],
                                                          ["8", "Name?", "Alice", _png()]])
    ds = ed.build_eval_dataset("docvqa_val", str(p), decode_images=False)
    s = list(ds.samples())
    assert s[0]["answer"] == ["42", "forty two"] and s[1]["answer"] == "Alice"
    assert s[0]["messages"][-1]["value"].endswith("single word or phrase.")
    res = evaluate(lambda smp: {"7": "forty two", "8": "Alise"}[smp["index"]], ds.samples(), ed.DEFAULT_METRIC[ds.kind])
    assert 0.85 < res["accuracy"] < 1.0 and res["n"] == 2             # one exact hit, one near miss (edit distance 1 of 5)
    try:
        ed.build_eval_dataset("nope", str(p))
        raise AssertionError
    except ValueError:
        pass
