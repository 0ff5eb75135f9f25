"""The host side of the attention kernels' launch plan (no GPU): which requests go to which
kernel, and how many splits the short ones get."""
from atom_b200 import native

SMS = 148


def test_requests_are_sorted_to_their_kernels():
    # group 4: 1 token = 4 packed rows (short), 5 tokens = 20 rows (mid: one 64-row tile), 200 tokens = 800 rows
    tiles, short, splits = native.flash_plan([1, 5, 200, 4, 0], 4, 8, 4096, sms=SMS)
    assert short and tiles == 1 + 13                       # 20 rows -> 1 tile, 800 rows -> 13 tiles; 16 rows are short
    tiles, short, splits, long_tiles = native.flash_plan([1, 5, 200, 4, 0], 4, 8, 4096, sms=SMS, long_rows=128)
    assert short and tiles == 1 and long_tiles == 7        # 800 rows -> 7 tiles of 128 on the tcgen05 kernel
    assert native.flash_plan([40, 40], 4, 8, 64, sms=SMS)[1] is False


def test_splits_fill_one_wave_but_stay_long_enough():
    # batch 8, 8 kv heads: 64 (request, kv head) pairs; two CTAs an SM -> 296 slots -> 4 splits
    assert native.flash_plan([1] * 8, 4, 8, 4096, sms=SMS)[2] == 4
    # batch 1: 8 pairs -> up to 37 splits, but no split shorter than 256 keys
    assert native.flash_plan([1], 4, 8, 4096, sms=SMS)[2] == 16
    assert native.flash_plan([1], 4, 8, 300, sms=SMS)[2] == 2
    assert native.flash_plan([1], 4, 8, 100, sms=SMS)[2] == 1
    # batch 64: more pairs than slots: more splits only where they fill whole waves much better
    assert native.flash_plan([1] * 64, 4, 8, 4096, sms=SMS)[2] == 1
    assert 1 <= native.flash_plan([1] * 40, 4, 8, 4096, sms=SMS)[2] <= 8
    assert native.flash_plan([1] * 8, 4, 8, 1 << 20, sms=SMS)[2] <= 64


def test_a_plan_for_any_batch_of_a_shape_covers_every_batch_of_it():
    """A step recorded once for (tokens, requests) is replayed for batches of any makeup within that
    shape: its tile counts must be no smaller than what any such batch needs, and it always provides
    for short requests."""
    import random
    rng = random.Random(5)
    for group, long_rows in ((1, 128), (4, 128), (8, 128), (4, 0), (16, 128), (3, 0)):
        for tokens, seqs in ((16, 8), (48, 8), (128, 8), (128, 32), (96, 64), (128, 64)):
            bound = native.flash_plan_for_any(tokens, seqs, group, 8, 4096, sms=SMS, long_rows=long_rows)
            assert bound[1] is True
            makeups = [[tokens], [1] * min(seqs, tokens), [tokens - 1, 1], [tokens // 2, tokens - tokens // 2]]
            for _ in range(200):
                n = rng.randint(1, min(seqs, tokens))
                cuts = sorted(rng.sample(range(1, tokens), n - 1)) if n > 1 else []
                lens = [b - a for a, b in zip([0] + cuts, cuts + [tokens])]
                if rng.random() < 0.5:      # not every token of the shape is used
                    lens = [max(0, x - rng.randint(0, 3)) for x in lens]
                makeups.append(lens)
            for lens in makeups:
                plan = native.flash_plan(lens, group, 8, 4096, sms=SMS, long_rows=long_rows)
                assert plan[0] <= bound[0], (group, long_rows, tokens, seqs, lens, plan, bound)
                if long_rows:
                    assert plan[3] <= bound[3], (group, long_rows, tokens, seqs, lens, plan, bound)


def test_where_the_gated_product_of_a_portion_runs_on_the_kernel_with_two_ctas_to_a_tile(monkeypatch):
    """How well a product's tiles (256 rows x 256 outputs, one pair of CTAs each) fill the rounds of 74 pairs,
    the ragged last round counting 0.72 where it is handed out in halves, and the rule built on it."""
    from atom_b200.parts import linear

    monkeypatch.setattr(native, "_pairs_resident", 74)
    monkeypatch.setattr(native, "gemm_pairs_supports", lambda M, N, K, lda, ldc: K % 8 == 0 and N % 8 == 0)
    # 2,048 rows x 12,288 outputs: 8 x 48 = 384 tiles = 5 rounds and 14 tiles, those in halves
    assert abs(native.gemm_pairs_waves(2048, 12288, True) - 384 / (5.72 * 74)) < 1e-9
    # 512 rows: 96 tiles = one round and 22 tiles in halves; 640 rows: 144 tiles = two rounds but four tiles
    assert abs(native.gemm_pairs_waves(512, 12288, True) - 96 / (1.72 * 74)) < 1e-9
    assert abs(native.gemm_pairs_waves(640, 12288, True) - 144 / (2 * 74)) < 1e-9
    # fewer tiles than pairs: one round, however few
    assert abs(native.gemm_pairs_waves(64, 4096, False) - 8 / 74) < 1e-9
    assert linear.pairs_pay(2048, 12288, 4096, 4096, 12288)
    assert linear.pairs_pay(640, 12288, 4096, 4096, 12288)
    assert not linear.pairs_pay(512, 12288, 4096, 4096, 12288)       # fills too little
    assert not linear.pairs_pay(64, 12288, 4096, 4096, 12288)        # too few rows
    assert not linear.pairs_pay(2048, 12288, 4100, 4100, 12288)      # a width the kernel refuses
    monkeypatch.setattr(linear, "PAIRS_MIN_ROWS", 0)
    assert not linear.pairs_pay(2048, 12288, 4096, 4096, 12288)      # switched off
    monkeypatch.setattr(native, "_pairs_resident", 0)                # the kernel cannot run on this device
    assert native.gemm_pairs_waves(2048, 12288, True) == 0.0
