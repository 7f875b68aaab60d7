"""Tile schedule of the fused expert-FFN kernel (csrc/kernels/moe_ffn.cu), checked on the host: the sequences of all CTAs cover
every tile of both phases exactly once, every CTA finishes its phase-0 tiles before its first phase-1 tile, and the CTAs' costs
stay level."""
import ctypes

import pytest

from gemm_b200 import _native


def _sequences(blocks, hidden, inter, grid):
    lib = _native.cuda()
    cap = 4096
    buf = (ctypes.c_int * (3 * cap))()
    out = []
    for c in range(grid):
        n = lib.gb_moe_ffn_schedule(blocks, hidden, inter, grid, c, buf, cap)
        assert 0 <= n <= cap
        out.append([(buf[3 * i], buf[3 * i + 1], buf[3 * i + 2]) for i in range(n)])
    return out


@pytest.mark.parametrize("blocks,hidden,inter,grid", [(128, 2048, 768, 148), (140, 2048, 768, 148), (16, 2048, 768, 148), (1, 256, 128, 148),
                                                      (37, 4096, 1536, 132), (148, 2048, 768, 148), (3, 2048, 768, 4)])
def test_schedule_covers_every_tile_once(blocks, hidden, inter, grid):
    seqs = _sequences(blocks, hidden, inter, grid)
    nb1, nb2 = inter // 128, hidden // 256
    seen = {}
    for c, seq in enumerate(seqs):
        phases = [t[0] for t in seq]
        assert phases == sorted(phases), f"CTA {c} interleaves the phases"
        for t in seq:
            assert t not in seen, f"tile {t} given to CTAs {seen[t]} and {c}"
            seen[t] = c
    want = {(0, b, n) for b in range(blocks) for n in range(nb1)} | {(1, b, n) for b in range(blocks) for n in range(nb2)}
    assert set(seen) == want
    # cost in k-steps: phase 0 tiles take hidden / 128, phase 1 tiles inter / 128; no CTA is more than about one phase-0 tile
    # above the mean (the granularity of the work)
    cost = [sum(hidden // 128 if t[0] == 0 else inter // 128 for t in seq) for seq in seqs]
    mean = sum(cost) / len(cost)
    assert max(cost) <= mean + hidden // 128 + inter // 128


def test_less_than_one_round_of_phase_0_spreads_phase_1_over_all_ctas():
    """One expert-parallel rank of eight: 16 token blocks give 96 gate/up tiles for 148 CTAs.  Every down tile has to wait for
    them anyway, so the down tiles go round-robin over ALL CTAs (one each), not only to the 52 CTAs without a gate/up tile."""
    seqs = _sequences(16, 2048, 768, 148)
    per_cta = [sum(1 for t in seq if t[0] == 1) for seq in seqs]
    assert max(per_cta) == 1 and sum(per_cta) == 16 * 8
    # with at least one full round of phase 0 the CTAs without the extra tile do run ahead
    seqs = _sequences(32, 2048, 768, 148)                     # 192 gate/up tiles: 44 CTAs take two
    heavy = [sum(1 for t in seq if t[0] == 1) for seq in seqs[:44]]
    light = [sum(1 for t in seq if t[0] == 1) for seq in seqs[44:]]
    assert max(heavy) < min(light)
