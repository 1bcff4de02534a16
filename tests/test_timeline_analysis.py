"""The host-side analysis of device timeline records (no GPU needed: synthetic records)."""
import numpy as np

from mccl_b200.utils import timeline as tl


def _recs():
    rows = []
    for c in range(4):      # GEMM launch A: four CTAs, 1 us .. 11 us
        rows.append([1000 + c * 10, 11000, tl.KIND_GEMM, (32 << 16) | 4, c, c])
    for c in range(4):      # GEMM launch B: another shape, 13 us .. 21 us
        rows.append([13000 + c * 10, 21000, tl.KIND_GEMM, (32 << 16) | 8, c, c])
    for c in range(2):      # an allreduce on two SMs of its own, 6 us .. 16 us
        rows.append([6000, 16000, tl.KIND_ALLREDUCE, 2, 100 + c, c])
    return np.array(sorted(rows), dtype=np.int64)


def test_overlap_figures():
    a = tl.analyze(_recs())
    assert abs(a["span_us"] - 20.0) < 1e-9 and a["gemm_launches"] == 2
    assert abs(a["gemm_busy_us"] - 18.0) < 1e-9
    assert abs(a["collective_busy_us"] - 10.0) < 1e-9
    assert abs(a["collective_not_under_gemm_us"] - 2.0) < 1e-9      # 11 us .. 13 us: no GEMM was running
    (c,) = a["collectives"]
    assert c["kind"] == "allreduce" and c["ctas"] == 2 and c["sms"] == 2
    assert abs(c["gemm_overlap"] - 0.8) < 1e-9 and c["ctas_sharing_sm_with_gemm"] == 0


def test_gemm_shapes_and_text():
    shapes = tl.gemm_shapes(_recs())
    assert [(s["m_tiles"], s["n_tiles_x_splits"], s["launches"], s["ctas"]) for s in shapes] == [(32, 4, 1, 4), (32, 8, 1, 4)]
    assert abs(shapes[0]["mean_us"] - 10.0) < 1e-9
    text = tl.summarize(_recs(), shapes=True)
    assert "GEMM busy 18.0 us in 2 launches" in text and "GEMM shapes" in text
    assert tl.analyze(np.zeros((0, 6), dtype=np.int64))["span_us"] == 0.0
