"""The softmax bookkeeping of the prefill attention kernel with two query tiles, restated in a few lines on the CPU:
a row's reference maximum moves only when the row's maximum has outgrown it by more than 8 (in powers of two), and
then the output accumulated so far and the sum are scaled to the new reference.  P may reach 256 meanwhile.  The
restatement rounds P to bfloat16 as the kernel does and must give the softmax of the whole row."""
import math

import pytest
import torch

STEP = 8.0     # inferrs_b200/csrc/attention_pair_tcgen05.cu: RESCALE_STEP
KEYS = 64


def lazily_rescaled(scores: torch.Tensor, values: torch.Tensor, scale: float):
    """scores [rows, keys] (raw), values [keys, d]: the kernel's walk over key tiles of 64, in float32."""
    rows, n = scores.shape
    scale_log2 = scale * math.log2(math.e)
    m_ref = torch.full((rows,), -math.inf)
    l = torch.zeros(rows)
    o = torch.zeros(rows, values.shape[1])
    moves = 0
    for k0 in range(0, n, KEYS):
        s = scores[:, k0:k0 + KEYS]
        mx = s.max(dim=1).values * scale_log2
        move = (mx > m_ref + STEP) | (torch.isinf(m_ref) & ~torch.isinf(mx))
        corr = torch.where(move, torch.where(torch.isinf(m_ref), torch.zeros(rows), torch.exp2(m_ref - mx)), torch.ones(rows))
        if k0 > 0:
            o *= corr[:, None]
            l *= corr
        moves += int(move.sum())
        m_ref = torch.where(move, mx, m_ref)
        m_safe = torch.where(torch.isinf(m_ref), torch.zeros(rows), m_ref)
        p = torch.exp2(s * scale_log2 - m_safe[:, None])
        l += p.sum(dim=1)
        o += p.to(torch.bfloat16).float() @ values[k0:k0 + KEYS]
    return o / l[:, None], moves, p.max()


@pytest.mark.parametrize("seed,spread", [(0, 1.0), (1, 6.0), (2, 20.0)])
def test_a_reference_that_moves_rarely_gives_the_same_softmax(seed, spread):
    g = torch.Generator().manual_seed(seed)
    rows, n, d = 32, 1024, 128
    scores = torch.randn(rows, n, generator=g) * spread
    scores[3, 700] = 60.0 * spread          # a late key that outgrows everything before it
    scores[5, :64] = -math.inf                # a row whose first tile is masked altogether
    values = torch.randn(n, d, generator=g).to(torch.bfloat16).float()
    scale = 0.35
    got, moves, _ = lazily_rescaled(scores, values, scale)
    p = torch.softmax(scores.double() * scale, dim=1)
    want = (p @ values.double()).float()
    assert not torch.isnan(got).any()
    err = (got - want).abs().max() / want.abs().max()
    assert err < 4e-3, err                     # P is rounded to bfloat16: eight bits
    # the reference moved far less often than the maximum grew (that is the point), but it did move
    tiles = n // KEYS
    assert rows <= moves < rows * tiles / 2


def test_p_stays_within_what_bfloat16_holds():
    """Between two moves a score may exceed the reference by at most the step: P is at most 2^8."""
    g = torch.Generator().manual_seed(7)
    scores = torch.cumsum(torch.rand(8, 640, generator=g) * 0.4, dim=1)   # ever growing rows
    values = torch.randn(640, 16, generator=g)
    _, moves, _ = lazily_rescaled(scores, values, 1.0)
    assert moves > 8
    # within a tile P is bounded by 2^(growth inside the tile + step)
    scale_log2 = math.log2(math.e)
    growth = (scores[:, 63::64] - scores[:, 0::64]).max() * scale_log2
    assert 2.0 ** (STEP + float(growth)) < 3.0e38
