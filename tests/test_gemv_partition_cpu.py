"""Integer model of the small-token kernel's work split, checked exhaustively on the CPU.

The kernel (csrc/nvfp4_gemv.cu) cuts the block space of each k-slab into equal contiguous
spans per CTA and per warp and combines split row groups through warp slots, CTA
contributions and arrival counters. This file restates that arithmetic and proves, for
many shapes and SM counts, that every weight block is consumed exactly once and that each
row group receives exactly the number of contributions its arrival counter waits for.
"""
import pytest

WARPS, MAX_SLAB = 16, 40


def geometry(rows, cols, pair, sms):
    groups = rows // 16 if pair else rows // 32
    kb = cols // 128
    slabs = (kb + MAX_SLAB - 1) // MAX_SLAB
    per_slab = max(sms // slabs, 1)
    # one slab: spans are cut at row-group boundaries (unit = blocks per group) while the imbalance that costs,
    # in blocks per CTA, stays below the price of a cross-CTA combine (48 blocks)
    aligned = False
    if slabs == 1:
        ctas = min(per_slab, groups)
        most = (groups + ctas - 1) // ctas
        aligned = (most * sms - groups) * kb <= 48 * sms
    unit = kb if aligned else 1
    per_slab = min(per_slab, groups * (kb // slabs) // unit)
    max_contrib = slabs * ((per_slab + groups - 1) // groups + 1)
    return groups, kb, slabs, per_slab, max_contrib, unit


def span_of(at, total, parts):
    return ((at + 1) * parts - 1) // total


def contributors(groups, kb, slabs, per_slab, unit, group):
    """(total, {(slab, cta): slot}) exactly as `contribute` computes them."""
    total, slots = 0, {}
    for s in range(slabs):
        kbs = (s + 1) * kb // slabs - s * kb // slabs
        units = groups * kbs // unit
        first = span_of(group * kbs // unit, units, per_slab)
        last = span_of(((group + 1) * kbs - 1) // unit, units, per_slab)
        for cta in range(first, last + 1):
            slots[(s, cta)] = total + (cta - first)
        total += last - first + 1
    return total, slots


def simulate(rows, cols, pair, sms):
    groups, kb, slabs, per_slab, max_contrib, unit = geometry(rows, cols, pair, sms)
    assert per_slab >= 1
    consumed = {}
    contributions = {}   # group -> list of (slab, cta)
    for s in range(slabs):
        kb_lo = s * kb // slabs
        kbs = (s + 1) * kb // slabs - kb_lo
        assert 1 <= kbs <= MAX_SLAB
        units = groups * kbs // unit
        for cta in range(per_slab):
            c0, c1 = cta * units // per_slab * unit, (cta + 1) * units // per_slab * unit
            length = c1 - c0
            assert length >= 1
            partial = {}          # (warp, slot) -> group
            direct = []
            for w in range(WARPS):
                w0, w1 = c0 + w * length // WARPS, c0 + (w + 1) * length // WARPS
                if w1 == w0:
                    continue
                first_group = w0 // kbs
                seg_group, seg_first = first_group, w0 % kbs

                def flush(group, first_kbi, last_kbi):
                    if first_kbi == 0 and last_kbi + 1 == kbs:
                        direct.append(group)
                    else:
                        slot = 0 if group == first_group else 1
                        assert (w, slot) not in partial
                        partial[(w, slot)] = group

                for at in range(w0, w1):
                    group, kbi = at // kbs, at % kbs
                    if group != seg_group:
                        flush(seg_group, seg_first, kbs - 1)
                        seg_group, seg_first = group, 0
                    key = (group, kb_lo + kbi)
                    assert key not in consumed
                    consumed[key] = (s, cta, w)
                flush(seg_group, seg_first, (w1 - 1) % kbs)
            # CTA-level assembly
            assembled = []
            first, count = c0 // kbs, (c1 - 1) // kbs - c0 // kbs + 1
            for index in range(count):
                group = first + index
                lo, hi = max(group * kbs, c0), min((group + 1) * kbs, c1)
                w_lo, w_hi = span_of(lo - c0, length, WARPS), span_of(hi - 1 - c0, length, WARPS)
                if w_lo == w_hi and lo == group * kbs and hi == (group + 1) * kbs:
                    assert group in direct
                    continue
                used = 0
                for w in range(w_lo, w_hi + 1):
                    b0, b1 = c0 + w * length // WARPS, c0 + (w + 1) * length // WARPS
                    if b1 == b0:
                        continue
                    slot = 0 if b0 // kbs == group else 1
                    assert partial.pop((w, slot)) == group
                    used += 1
                assert used >= 1
                assembled.append(group)
            assert not partial, "a warp partial was never combined"
            for group in direct + assembled:
                contributions.setdefault(group, []).append((s, cta))
    assert len(consumed) == groups * kb
    for group in range(groups):
        total, slots = contributors(groups, kb, slabs, per_slab, unit, group)
        if unit > 1:
            assert total == 1
        got = contributions.get(group, [])
        assert len(got) == total == len(set(got)), (group, total, got)
        assert total <= max_contrib
        assert sorted(slots[c] for c in got) == list(range(total))


@pytest.mark.parametrize("rows,cols,pair", [
    (17408, 5120, False), (17408, 5120, True), (5120, 17408, False), (10240, 5120, False), (5120, 5120, False),
    (5120, 10240, False), (2176, 5120, True), (5120, 2176, False), (4352, 5120, True), (5120, 4352, False),
    (32, 128, False), (16, 128, True), (64, 256, False), (128, 17408, False), (96, 640, False), (48, 5120, True),
    (32, 5248, False), (6144, 5120, False)])
@pytest.mark.parametrize("sms", [148, 132, 7, 1])
def test_every_block_once_and_counters_match(rows, cols, pair, sms):
    simulate(rows, cols, pair, sms)


# ---- pair-tile GEMM: leftover tiles cut along k (csrc/nvfp4_gemm.cu, pair_work) -----------------------------
SPLIT_WAYS = 8


def pair_geometry(tiles, sm_pairs, k_blocks):
    """(pairs launched, pairs that share the leftover tiles) as the host side picks them; sharers 0: whole tiles only."""
    pairs = min(tiles, sm_pairs)
    left = tiles % sm_pairs
    sharers = min(left * SPLIT_WAYS, sm_pairs, left * k_blocks)
    if left == 0 or sharers <= left:
        return pairs, 0
    return max(pairs, sharers), sharers


def pair_work(pair, pairs, tiles, k_blocks, sharers):
    """The items of one CTA pair in the order the kernel does them: (tile, kb0, kb1, kind, first_giver)."""
    if not sharers:
        return [(tile, 0, k_blocks, 0, 0) for tile in range(pair, tiles, pairs)]
    whole = tiles // pairs
    items = [(pair + i * pairs, 0, k_blocks, 0, 0) for i in range(whole)]
    if pair >= sharers:
        return items
    first_left = whole * pairs
    units = (tiles - first_left) * k_blocks
    x0, x1 = pair * units // sharers, (pair + 1) * units // sharers
    assert x1 > x0
    a, b = x0 // k_blocks, (x1 - 1) // k_blocks
    a_begin, a_end = a * k_blocks, (a + 1) * k_blocks
    given = finishing = None
    if x1 >= a_end:
        first_giver = ((a_begin + 1) * sharers - 1) // units
        finishing = (first_left + a, x0 - a_begin, k_blocks, 0 if first_giver == pair else 2, first_giver)
    else:
        given = (first_left + a, x0 - a_begin, x1 - a_begin, 1, 0)
    if b > a:
        assert given is None
        given = (first_left + b, 0, x1 - b * k_blocks, 1, 0)
    return ([given] if given else []) + ([finishing] if finishing else []) + items


@pytest.mark.parametrize("tiles,sm_pairs,k_blocks", [(320, 74, 68), (80, 74, 13), (80, 74, 20), (272, 74, 20), (1088, 74, 20),
                                                     (75, 74, 74), (147, 74, 2), (5, 2, 7), (9, 4, 5), (320, 66, 34), (20, 74, 68),
                                                     (1, 74, 80), (73, 74, 2), (2, 74, 20), (80, 74, 1), (148, 74, 20), (3, 74, 3)])
def test_pair_tile_leftover_split(tiles, sm_pairs, k_blocks):
    pairs, sharers = pair_geometry(tiles, sm_pairs, k_blocks)
    assert pairs <= sm_pairs
    done, givers, finisher, load = {}, {}, {}, []
    for pair in range(pairs):
        items = pair_work(pair, pairs, tiles, k_blocks, sharers)
        kinds = [item[3] for item in items]
        assert kinds.count(1) <= 1 and kinds.count(2) <= 1
        assert all(k != 1 for k in kinds[1:]) and all(k != 2 for k in kinds[2:])    # handed-over first, finishing next
        assert 2 not in kinds[1:] or kinds[0] == 1
        blocks = 0
        for tile, kb0, kb1, kind, first_giver in items:
            assert 0 <= kb0 < kb1 <= k_blocks
            for kb in range(kb0, kb1):
                assert (tile, kb) not in done
                done[(tile, kb)] = pair
            blocks += kb1 - kb0
            if kind == 1:
                givers.setdefault(tile, []).append(pair)
            elif kind == 2:
                finisher[tile] = (pair, first_giver)
            else:
                assert kb0 == 0 and kb1 == k_blocks, "a partial item must hand over or finish"
        load.append(blocks)
    assert len(done) == tiles * k_blocks
    if sharers:
        assert max(load[:sharers]) - min(load[:sharers]) <= 1     # the sharers issue the same number of k blocks
        assert sharers == pairs or max(load[sharers:]) <= min(load[:sharers])
    for tile, who in givers.items():
        pair, first_giver = finisher[tile]
        assert who == list(range(first_giver, pair))  # exactly the pairs the finisher waits for, in order
        assert len(who) < SPLIT_WAYS + 1
    for tile, (pair, first_giver) in finisher.items():
        assert first_giver < pair and tile in givers
