"""Device timeline: where kernels ran, read from stamps the kernels wrote themselves.

The GEMM and collective kernels of this package can stamp ``%globaltimer`` at
entry and exit of each CTA into a device buffer (``csrc/core/timeline.hpp``).
That shows, without a profiler, whether a gradient allreduce really ran beside
the backward GEMMs of a replayed CUDA graph, on which SMs, and for how long.

    from mccl_b200.utils import timeline
    timeline.enable(device_index)        # before the CUDA graph is captured
    ... run one step, synchronize ...
    recs = timeline.drain(device_index)  # numpy [n, 6]: t0, t1, kind, tag, sm, cta
    print(timeline.summarize(recs))
"""
from __future__ import annotations

from typing import Dict, List

import numpy as np

from .. import _C

KIND_GEMM, KIND_ALLREDUCE, KIND_OTHER_COLL, KIND_OP, KIND_GEMM_PHASE = 1, 2, 3, 4, 5
_KIND_NAME = {KIND_GEMM: "gemm", KIND_ALLREDUCE: "allreduce", KIND_OTHER_COLL: "collective", KIND_OP: "op"}


def enable(device: int, capacity: int = 1 << 17, every: int = 1, detail: bool = False) -> None:
    """Starts recording on ``device``; CTAs whose index is a multiple of ``every`` record.  With ``detail`` the GEMM
    kernel also records its inner phases per tile (kind 5: set-up, wait for the accumulator, epilogue)."""
    _C.timeline_enable(device, capacity, every, 1 if detail else 0)


def disable(device: int) -> None:
    _C.timeline_disable(device)


def drain(device: int) -> np.ndarray:
    """Synchronises the device and returns (and forgets) the records so far, sorted by start time."""
    return _C.timeline_drain(device).numpy()


def _union_length(intervals: np.ndarray) -> int:
    """Total length covered by [t0, t1) intervals (sorted by t0)."""
    if len(intervals) == 0:
        return 0
    total, cur0, cur1 = 0, int(intervals[0, 0]), int(intervals[0, 1])
    for t0, t1 in intervals[1:]:
        if t0 > cur1:
            total += cur1 - cur0
            cur0, cur1 = int(t0), int(t1)
        else:
            cur1 = max(cur1, int(t1))
    return total + cur1 - cur0


def _launches(recs: np.ndarray, gap_ns: int = 1500) -> List[np.ndarray]:
    """Groups CTA records of one kind into kernel launches: same tag, start times within gap_ns of the group."""
    out: List[np.ndarray] = []
    if len(recs) == 0:
        return out
    start = 0
    for i in range(1, len(recs) + 1):
        if i == len(recs) or recs[i, 3] != recs[start, 3] or recs[i, 0] > recs[start:i, 1].max() + gap_ns:
            out.append(recs[start:i])
            start = i
    return out


def analyze(recs: np.ndarray) -> Dict:
    """Per-collective overlap figures of the records of ONE step."""
    if len(recs) == 0:
        return {"span_us": 0.0, "collectives": [], "gemm_busy_us": 0.0}
    t_begin, t_end = int(recs[:, 0].min()), int(recs[:, 1].max())
    gemm = recs[recs[:, 2] == KIND_GEMM]
    coll = recs[(recs[:, 2] == KIND_ALLREDUCE) | (recs[:, 2] == KIND_OTHER_COLL)]
    gemm_iv = gemm[:, :2]
    rows = []
    for k in _launches(coll):
        k0, k1 = int(k[:, 0].min()), int(k[:, 1].max())
        # GEMM activity (any CTA) clipped to the collective's lifetime
        g = gemm_iv[(gemm_iv[:, 1] > k0) & (gemm_iv[:, 0] < k1)].copy()
        g[:, 0] = np.maximum(g[:, 0], k0)
        g[:, 1] = np.minimum(g[:, 1], k1)
        covered = _union_length(g[np.argsort(g[:, 0])]) if len(g) else 0
        # SMs the collective's CTAs shared with a GEMM CTA at the same time
        shared = 0
        for t0, t1, _, _, sm, _ in k:
            m = (gemm[:, 4] == sm) & (gemm[:, 1] > t0) & (gemm[:, 0] < t1)
            shared += int(m.any())
        rows.append({
            "kind": _KIND_NAME.get(int(k[0, 2]), "?"),
            "start_us": (k0 - t_begin) / 1e3,
            "dur_us": (k1 - k0) / 1e3,
            "ctas": int(len(k)),
            "sms": int(len(set(k[:, 4].tolist()))),
            "gemm_overlap": covered / max(k1 - k0, 1),
            "ctas_sharing_sm_with_gemm": shared,
        })
    g_sorted = gemm_iv[np.argsort(gemm_iv[:, 0])] if len(gemm_iv) else gemm_iv
    c_iv = coll[:, :2]
    c_sorted = c_iv[np.argsort(c_iv[:, 0])] if len(c_iv) else c_iv
    # time during which a collective ran and no GEMM did: the exposed part (other operators aside)
    exposed = 0
    if len(c_sorted):
        both = np.concatenate([g_sorted, c_sorted]) if len(g_sorted) else c_sorted
        both = both[np.argsort(both[:, 0])]
        exposed = _union_length(both) - _union_length(g_sorted)
    return {
        "span_us": (t_end - t_begin) / 1e3,
        "gemm_busy_us": _union_length(g_sorted) / 1e3,
        "gemm_launches": len(_launches(gemm[np.argsort(gemm[:, 0])])) if len(gemm) else 0,
        "collective_busy_us": _union_length(c_sorted) / 1e3,
        "collective_not_under_gemm_us": exposed / 1e3,
        "collectives": rows,
    }


def gemm_shapes(recs: np.ndarray) -> List[Dict]:
    """Per GEMM launch shape (m tiles, n tiles x k splits): launches, CTAs, and time from the first CTA's start
    to the last CTA's end, as the kernels themselves saw it inside the running step."""
    gemm = recs[recs[:, 2] == KIND_GEMM]
    if len(gemm) == 0:
        return []
    gemm = gemm[np.argsort(gemm[:, 0])]
    by_shape: Dict[int, List] = {}
    for k in _launches(gemm):
        by_shape.setdefault(int(k[0, 3]), []).append((int(k[:, 1].max() - k[:, 0].min()), len(k),
                                                       float((k[:, 1] - k[:, 0]).mean())))
    rows = []
    for tag, v in by_shape.items():
        rows.append({"m_tiles": tag >> 16, "n_tiles_x_splits": tag & 0xffff, "launches": len(v),
                     "ctas": v[0][1], "mean_us": sum(x[0] for x in v) / len(v) / 1e3,
                     "total_us": sum(x[0] for x in v) / 1e3, "mean_cta_us": sum(x[2] for x in v) / len(v) / 1e3})
    rows.sort(key=lambda r: -r["total_us"])
    return rows


def summarize(recs: np.ndarray, shapes: bool = False) -> str:
    a = analyze(recs)
    lines = [f"span {a['span_us']:.1f} us; GEMM busy {a['gemm_busy_us']:.1f} us in {a.get('gemm_launches', 0)} launches; "
             f"collectives busy {a.get('collective_busy_us', 0.0):.1f} us, of which {a.get('collective_not_under_gemm_us', 0.0):.1f} us "
             f"with no GEMM running"]
    lines.append("  kind        start_us   dur_us  ctas  sms  gemm_overlap  ctas_on_gemm_sm")
    for r in a["collectives"]:
        lines.append(f"  {r['kind']:<10} {r['start_us']:9.1f} {r['dur_us']:8.1f} {r['ctas']:5d} {r['sms']:4d} "
                     f"{r['gemm_overlap']:12.2f} {r['ctas_sharing_sm_with_gemm']:16d}")
    if shapes:
        lines.append("  GEMM shapes: m_tiles  n_tiles*splits  launches  ctas  mean_us  mean_cta_us  total_us")
        for r in gemm_shapes(recs):
            lines.append(f"    {r['m_tiles']:6d} {r['n_tiles_x_splits']:8d} {r['launches']:9d} {r['ctas']:5d} {r['mean_us']:8.1f} "
                         f"{r['mean_cta_us']:11.1f} {r['total_us']:9.1f}")
    return "\n".join(lines)
