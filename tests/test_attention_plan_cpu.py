"""Host-side planning of the decode attention kernel's stream-K work list (ops/attention.py::build_work_streamk)."""
from gemm_b200.ops import attention as att


def test_stream_k_plan_covers_every_item_once():
    for lens, hkv, n in (([2049] * 64, 4, 296), ([17, 900, 4000, 128, 129], 2, 296), ([300] * 8, 8, 50)):
        work, splits = att.build_work_streamk(lens, hkv, n_cta=n)
        cover = {}
        for c in range(work.shape[0]):
            for f in range(work.shape[1]):
                seq, packed, lo, hi = work[c, f].tolist()
                if seq < 0:
                    break
                cover.setdefault((seq, packed & 0xff), []).append(((packed >> 8) & 0xff, (packed >> 16) & 0xff, lo, hi))
        assert len(cover) == len(lens) * hkv
        for v in cover.values():
            v.sort()
            assert [x[0] for x in v] == list(range(len(v))) and all(x[1] == len(v) for x in v) and len(v) <= splits
            assert v[0][2] == 0 and v[-1][3] == 65536 and all(v[i][3] == v[i + 1][2] for i in range(len(v) - 1))
    assert att.build_work_streamk([5] * 300, 4) is None       # many one-block items: more fragments per CTA than the kernel holds
