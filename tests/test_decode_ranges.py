"""The arithmetic by which the decode attention deals its key tiles over the blocks, restated on the host.

The kernel (quanta_b200/csrc/attention_mma.cu, ``attn_decode_kernel``) lists the 64-key tiles of all
(token, kv head) pairs, token by token and head by head, and gives block ``b`` of ``A`` the tiles
``[b*T/A, (b+1)*T/A)``.  A pair that a boundary cuts leaves one partial result per block that holds some of
its tiles, numbered ``seg = b - first block of the pair``; the scratch has ``n_parts - 1`` entries a row
with ``n_parts = min(tiles of the longest context, 2*SMs/kv_heads + 2) + 1`` (``qb_attn_decode_parts``).
This test checks, for random batches, that the ranges cover every tile exactly once, that the kernel's
closed form for ``seg`` is the count of blocks since the pair's first tile, and that no pair ever needs
more entries than the scratch has: the figures a wrong result or a refused step would come from.
"""

import bisect
import random

BN = 64


def tiles_of(pos: int, window: int) -> int:
    lo = max(0, pos - window + 1) if window > 0 else 0
    return pos // BN - lo // BN + 1


def n_parts(nkv: int, max_len: int, sms: int) -> int:
    tiles = -(-max_len // BN)
    return min(tiles, 2 * sms // nkv + 2) + 1


def deal(positions, nkv, window, grid):
    """For each block its (pair, tile, seg) triples, computed as the kernel's producer does."""
    cum = [0]
    for p in positions:
        cum.append(cum[-1] + tiles_of(p, window))
    T = nkv * cum[-1]
    A = min(T, grid)
    out = []
    for b in range(grid):
        start, end = (b * T // A, (b + 1) * T // A) if b < A else (0, 0)
        mine = []
        for gt in range(start, end):
            a = bisect.bisect_right(cum, gt // nkv) - 1          # nkv * cum[a] <= gt < nkv * cum[a + 1]
            cnt = cum[a + 1] - cum[a]
            base = nkv * cum[a]
            kvh, i = divmod(gt - base, cnt)
            g0 = base + kvh * cnt
            seg = b - ((g0 + 1) * A - 1) // T
            mine.append(((a, kvh), i, seg))
        out.append(mine)
    return out, T


def test_ranges_cover_every_tile_once_and_segments_fit_the_scratch():
    rng = random.Random(0)
    for case in range(200):
        sms = rng.choice([4, 16, 132, 148])
        nkv = rng.choice([1, 2, 3, 8])
        n_dec = rng.choice([1, 2, 5, 8, 64, 200])
        window = rng.choice([0, 0, 100, 1000])
        longest = rng.choice([1, 63, 64, 65, 700, 5000] + ([140000] if n_dec <= 2 else []))
        positions = [rng.randrange(longest) for _ in range(n_dec)]
        blocks, T = deal(positions, nkv, window, sms)
        seen = {}
        first_block = {}
        for b, mine in enumerate(blocks):
            for pair, i, seg in mine:
                assert (pair, i) not in seen
                seen[pair, i] = b
                first_block.setdefault(pair, b)
                assert seg == b - first_block[pair] >= 0          # blocks since the one with the pair's first tile
        assert len(seen) == T == nkv * sum(tiles_of(p, window) for p in positions)
        # tiles of a pair lie in consecutive blocks, in order
        for (pair, i), b in seen.items():
            if i:
                assert seen[pair, i - 1] in (b - 1, b)
        limit = n_parts(nkv, max(positions) + 1, sms) - 1         # partial results a row can hold
        worst = max(seg for mine in blocks for _, _, seg in mine)
        assert worst < limit, (case, sms, nkv, n_dec, longest, worst, limit)
