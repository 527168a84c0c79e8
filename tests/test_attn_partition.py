"""The tile shares of the batched decode attention (csrc/attn_decode.cu, balanced grid), restated on the host: group c
of n_kv_heads CTAs takes tiles [c*Q, (c+1)*Q) of the 64-row tiles of all sequences numbered sequence by sequence, with
Q = max(ceil(total / groups), split_len / 64, ceil(longest / n_splits)).  Checked for random mixes of lengths: every
tile is taken exactly once, a sequence is cut into at most n_splits + 1 pieces (the scratch holds n_splits + 1 slots
per (sequence, KV head)), its pieces use the slots 0 .. n_used - 1 in order, and all of them agree on n_used."""
import random

TILE = 64


def partition(lens, groups, n_splits, split_len):
    tiles = [(l + TILE - 1) // TILE for l in lens]
    pre = [0]
    for t in tiles:
        pre.append(pre[-1] + t)
    total, longest = pre[-1], max(tiles)
    quota = max((total + groups - 1) // groups, max(max(split_len // TILE, 1), (longest + n_splits - 1) // n_splits))
    pieces = []  # (group, seq, first row, end row, slot, n_used)
    for grp in range(groups):
        t, t_end = grp * quota, min((grp + 1) * quota, total)
        seq = 0
        while t < t_end:
            while pre[seq + 1] <= t:
                seq += 1
            t_seq = pre[seq + 1] - pre[seq]
            j0 = t - pre[seq]
            j1 = min(t_seq, j0 + (t_end - t))
            first_grp, last_grp = pre[seq] // quota, (pre[seq + 1] - 1) // quota
            pieces.append((grp, seq, j0 * TILE, min(j1 * TILE, lens[seq]), grp - first_grp, last_grp - first_grp + 1))
            t += j1 - j0
    return pieces


def check(lens, groups, n_splits, split_len):
    pieces = partition(lens, groups, n_splits, split_len)
    for s, length in enumerate(lens):
        mine = sorted((p for p in pieces if p[1] == s), key=lambda p: p[2])
        assert mine, (s, lens)
        n_used = mine[0][5]
        assert len(mine) == n_used <= n_splits + 1, (lens, groups, n_splits, split_len, mine)
        assert [p[4] for p in mine] == list(range(n_used))
        assert all(p[5] == n_used for p in mine)
        assert mine[0][2] == 0 and mine[-1][3] == length
        for a, b in zip(mine, mine[1:]):
            assert a[3] == b[2] and a[3] % TILE == 0   # contiguous, cut at tile boundaries
        assert all(p[3] > p[2] for p in mine)


def test_every_tile_once_and_pieces_fit_the_slots():
    rng = random.Random(7)
    for _ in range(400):
        n_seqs = rng.randint(2, 256)
        max_len = rng.choice([1, 65, 700, 4224, 8192])
        lens = [rng.randint(1, max_len) for _ in range(n_seqs)]
        if rng.random() < 0.3:
            lens[rng.randrange(n_seqs)] = max_len
        split_len = rng.choice([32, 64, 128, 256, 1024])
        n_splits = max(1, (max(lens) + split_len - 1) // split_len)
        groups = rng.choice([1, 3, 55, 111, 444])
        check(lens, groups, n_splits, split_len)


def test_uniform_batch_of_the_benchmark():
    # 32 sequences at 1100 rows, 8 KV heads on 444 resident CTAs: 55 groups, quota 11 tiles
    pieces = partition([1100] * 32, 55, 5, 256)
    assert max(p[3] - p[2] for p in pieces) <= 11 * TILE
    assert len({p[0] for p in pieces}) == 53   # 576 tiles / 11 per group
