"""The markdown report writer on a hand-made record set (no GPU)."""
import json

from rocm_wmma_gemm_b200 import generate_report as gr


def _rec(m, la, lb, lc, tf, typ="f16_f16"):
    return {"type": typ, "M": m, "N": m, "K": m, "layout": {"A": la, "B": lb, "C": lc}, "tflops_median": tf,
            "tflops_graph": tf * 1.1}


def test_pivot_and_render(tmp_path):
    recs = [_rec(1024, 1, 1, 1, 100.0), _rec(1024, 1, 1, 0, 110.0), _rec(1024, 0, 1, 0, 90.0),
            _rec(1024, 0, 1, 0, 95.0), _rec(2048, 0, 0, 1, 700.0, "f32_bf16")]
    path = tmp_path / "r.jsonl"
    path.write_text("\n".join(json.dumps(r) for r in recs) + "\n")
    table = gr.pivot(gr.load_records([str(path)]))
    assert table[("f16_f16", 1024, 1024, 1024)][(1, 1)] == {1: 100.0, 0: 110.0}
    assert table[("f16_f16", 1024, 1024, 1024)][(0, 1)] == {0: 95.0}  # best of the repeats
    text = gr.render(table, "T", "B200", "median")
    assert "| 1024x1024x1024 | col, col | 100.00 | 110.00 | 4.9 |" in text
    assert "| 1024x1024x1024 | row, col | – | 95.00 | 4.2 |" in text
    assert "## BF16 -> F32 Performance Results" in text and "## F16 -> F16 Performance Results" in text
    out = tmp_path / "r.md"
    assert gr.main([str(path), "-o", str(out), "--metric", "tflops_graph", "--json-out", str(tmp_path / "r.json")]) == 0
    assert "110.00" in out.read_text()
    assert abs(json.loads((tmp_path / "r.json").read_text())[0]["C_col"] - 110.0) < 1e-9
