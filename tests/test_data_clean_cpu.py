"""Raw-corpus cleaning, list conversion and fixed-length packing (data/clean.py)."""
import json

import numpy as np

from linear_moe_b200.data import clean as C
from linear_moe_b200.data.datasets import IndexedDataset
from linear_moe_b200.data.tokenizer import NullTokenizer


def test_clean_text_rules():
    raw = "看  这里 https://example.com/a?b=1&c=%20d  很好！<b>bold</b>\t#tag【注】 50% (ok)"
    out = C.clean_text(raw)
    assert "http" not in out and "example" not in out
    assert "  " not in out and "<" not in out and "#" not in out and "【" not in out and "\t" not in out
    assert out.startswith("看 这里 很好！bbold/b") and out.endswith("50% (ok)")
    assert C.clean_text("   ") == ""


def test_clean_dir_pretrain_and_sft_layouts(tmp_path):
    src, dst, dst2 = tmp_path / "in", tmp_path / "out", tmp_path / "sft"
    src.mkdir()
    (src / "a.json").write_text(json.dumps([{"content": "第一 篇  http://x.y/z 文章。"}, {"title": "no text field"},
                                            {"output": "second @@ one"}], ensure_ascii=False), encoding="utf-8")
    (src / "b.jsonl").write_text('{"text": "line   one"}\n\n{"text": "x"}\n', encoding="utf-8")
    (src / "broken.json").write_text("[{not json", encoding="utf-8")
    assert C.clean_dir(str(src), str(dst), processes=2) == 4
    rows = [json.loads(l) for l in (dst / "a.json").read_text(encoding="utf-8").splitlines()]
    assert rows == [{"text": "第一 篇 文章。"}, {"text": "second one"}]
    assert (dst / "broken.json").read_text() == ""
    assert C.clean_dir(str(src), str(dst2), target_key="content", min_chars=2) == 3
    row = json.loads((dst2 / "b.jsonl").read_text(encoding="utf-8").splitlines()[0])
    assert row == {"instruction": "", "input": "", "content": "line one"}


def test_jsonl_to_list_in_place(tmp_path):
    f = tmp_path / "v.json"
    f.write_text('{"a": 1}\n{"a": 2}\n')
    assert C.jsonl_to_list(str(f)) == 2
    assert json.loads(f.read_text()) == [{"a": 1}, {"a": 2}]
    assert C.jsonl_to_list(str(f)) == 2                       # a list stays a list


def test_pack_concatenates_and_drops_the_tail(tmp_path):
    rows = C.pack_tokens([[1, 2, 3], [4, 5], [6, 7, 8, 9, 10, 11]], 4)
    assert [r.tolist() for r in rows] == [[1, 2, 3, 4], [5, 6, 7, 8]]
    src = tmp_path / "d.jsonl"
    src.write_text("\n".join(json.dumps({"text": " ".join(str(i) for i in range(k, k + 5))}) for k in (0, 10, 20)))
    n = C.pack_file(str(src), str(tmp_path / "packed"), NullTokenizer(100), 6, append_eod=True)
    assert n == 3
    ds = IndexedDataset(str(tmp_path / "packed"))
    assert len(ds) == 3 and all(ds.sizes == 6)
    assert np.concatenate([ds.get(i) for i in range(3)]).tolist() == [0, 1, 2, 3, 4, 99, 10, 11, 12, 13, 14, 99, 20, 21, 22, 23, 24, 99]
    C.main(["pack", "--input", str(src), "--output-prefix", str(tmp_path / "p2"), "--sequence-length", "5", "--vocab-size", "100"])
    assert len(IndexedDataset(str(tmp_path / "p2"))) == 3
