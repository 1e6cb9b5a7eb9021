"""The work split of the tensor-memory launch (csrc/nvfp4_gemv_tc.cu), checked on the CPU for many shapes and SM
counts through the host-side description entry: every (tile, k block) of every product is streamed exactly once,
by exactly one CTA; a tile's parts fill its contributor slots without a gap or a clash; the jobs partition the
input groups of their product; and a step marked `keeps` gives no CTA a second item. The item arithmetic restated
here is the kernel's (`cursor_load`): item i of a step belongs to CTA i mod ctas, tile = i / parts, part = i % parts,
k range [kb0 + part * span / parts, kb0 + (part + 1) * span / parts).
"""
from ctypes import byref

import pytest

from augur_v100_b200 import abi

SM_COUNTS = [1, 2, 7, 74, 132, 148, 160, 264, 512]
LINEARS = [(128, 64), (128, 256), (256, 1216), (2560, 2048), (5120, 5120), (10240, 5120), (5120, 10240), (17408, 5120),
           (5120, 17408), (5120, 2176), (248320 // 128 * 128, 5120), (384, 8192), (128, 30720)]
MLPS = [(256, 512), (1024, 2176), (640, 1152), (5120, 2176), (5120, 17408), (2048, 30080), (1024, 39552), (128, 34304),
        (3712, 24448), (4096, 128), (128, 128), (5120, 4352)]


def describe(rows_a, cols_a, epilogue_a, rows_b, cols_b, sms):
    out = abi.TcProgram()
    result = abi.lib().augur_cuda_nvfp4_sm100_tc_program_describe_host_v1(rows_a, cols_a, epilogue_a, rows_b, cols_b, sms, byref(out))
    assert result.status == abi.STATUS_OK, (rows_a, cols_a, rows_b, cols_b, sms, result.status)
    return out


def check_program(program, sms, products):
    """`products`: [(tiles, k_blocks, input_groups)] per phase."""
    ctas = program.ctas
    assert 1 <= ctas <= 2 * sms
    covered = [dict() for _ in products]          # phase -> {(tile, kb): count}
    slots = [dict() for _ in products]            # phase -> {tile: set of slots}
    for index in range(program.steps):
        step = program.step[index]
        tiles, k_blocks, _ = products[step.phase]
        assert step.tiles >= 1 and step.parts >= 1 and step.tile0 + step.tiles <= tiles
        assert step.kb0 < step.kb1 <= k_blocks and step.parts <= step.kb1 - step.kb0
        assert step.parts <= 16 and (step.parts == 1 or (step.kb1 - step.kb0) // step.parts >= 2)
        assert 1 <= step.job + 1 <= program.jobs and program.job[step.job].phase == step.phase
        items, span = step.tiles * step.parts, step.kb1 - step.kb0
        per_cta = {}
        for item in range(items):
            cta = item % ctas
            per_cta[cta] = per_cta.get(cta, 0) + 1
            tile, part = step.tile0 + item // step.parts, item % step.parts
            lo, hi = step.kb0 + part * span // step.parts, step.kb0 + (part + 1) * span // step.parts
            assert lo < hi
            for kb in range(lo, hi):
                covered[step.phase][(tile, kb)] = covered[step.phase].get((tile, kb), 0) + 1
            taken = slots[step.phase].setdefault(tile, set())
            assert step.slot0 + part not in taken
            taken.add(step.slot0 + part)
        if step.keeps:
            assert max(per_cta.values()) == 1 and step.parts == 1 and step.feeds
        if step.feeds:
            fed = program.job[step.feeds]
            assert step.parts == 1 and fed.phase == step.phase + 1
            # a gate|up tile of 128 physical rows is 64 columns of the intermediate: 4 groups of 16
            assert (fed.group0, fed.groups) == (step.tile0 * 4, step.tiles * 4)
    for phase, (tiles, k_blocks, groups) in enumerate(products):
        assert len(covered[phase]) == tiles * k_blocks and set(covered[phase].values()) == {1}
        for tile in range(tiles):
            assert slots[phase][tile] == set(range(program.contributors[phase]))
        mine = sorted((program.job[j].group0, program.job[j].groups) for j in range(program.jobs) if program.job[j].phase == phase)
        at = 0
        for group0, count in mine:
            assert group0 == at and count >= 1
            at += count
        assert at == groups
    # the k blocks a step streams hold exactly the groups of its job (16 groups of 16 per 256-deep block; a job's last
    # block may be ragged)
    for index in range(program.steps):
        step, job = program.step[index], program.job[program.step[index].job]
        assert step.kb0 * 16 == job.group0 and (step.kb1 - 1) * 16 < job.group0 + job.groups <= step.kb1 * 16


@pytest.mark.parametrize("sms", SM_COUNTS)
def test_linear_programs_cover_every_block_once(sms):
    for rows, cols in LINEARS:
        for epilogue in (abi.EPILOGUE_LINEAR_BF16, abi.EPILOGUE_SWIGLU_BF16):
            physical = rows * (2 if epilogue == abi.EPILOGUE_SWIGLU_BF16 else 1)
            if physical * cols >= 1 << 32 or physical // 128 * 8 > 16384:     # beyond the entries' index and counter ranges
                continue
            program = describe(rows, cols, epilogue, 0, 0, sms)
            assert program.steps == 1 and program.jobs == 1
            check_program(program, sms, [(physical // 128, (cols + 255) // 256, cols // 16)])
            assert program.ctas == min(physical // 128 * program.step[0].parts, 2 * sms)


@pytest.mark.parametrize("sms", SM_COUNTS)
def test_mlp_programs_cover_every_block_once(sms):
    for hidden, inter in MLPS:
        program = describe(inter, hidden, 0, hidden, inter, sms)
        tiles_a = 2 * inter // 128
        check_program(program, sms, [(tiles_a, (hidden + 255) // 256, hidden // 16), (hidden // 128, (inter + 255) // 256, inter // 16)])
        waves = sum(1 for i in range(program.steps) if program.step[i].phase == 0)
        assert program.steps == 2 * waves and waves in (1, 2)
        if waves == 2:      # more gate|up tiles than CTAs: the first wave fills the CTAs and ends on a k block of the second product
            assert tiles_a > 2 * sms and program.step[0].tiles % 4 == 0 and program.step[0].tiles <= 2 * sms
        else:
            assert tiles_a <= 2 * sms or (2 * sms) // 4 == 0


def test_description_rejects_what_the_entries_reject():
    out = abi.TcProgram()
    describe_raw = abi.lib().augur_cuda_nvfp4_sm100_tc_program_describe_host_v1
    for arguments in [(100, 64, 0, 0, 0, 148), (128, 96, 0, 0, 0, 148), (128, 64, 7, 0, 0, 148), (128, 64, 0, 0, 0, 0),
                      (128, 64, 0, 0, 0, 513), (0, 64, 0, 0, 0, 148), (17408, 5120, 0, 5120, 17344, 148),
                      (17408, 5120, 0, 5248, 17408, 148), (1 << 20, 8192, 0, 0, 0, 148)]:
        assert describe_raw(*arguments, byref(out)).status == abi.STATUS_INVALID_ARGUMENT, arguments
    assert describe_raw(128, 64, 0, 0, 0, 148, None).status == abi.STATUS_INVALID_ARGUMENT
