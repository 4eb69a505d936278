"""Host-side choices of the attention wrappers: which decode kernel a step takes, whether its decoding requests
get a kernel of their own, and how the keys of prompt tiles are divided among blocks.  Pure functions of the
step's lengths; the times quoted are measurements on a B200 (profiles/), the assertions say which of the
measured options the choice must be."""

from types import SimpleNamespace

import pytest

from yalis_b200.ops import attention as attn


def host(q_lens, before, **kw):
    starts = [0]
    for q in q_lens:
        starts.append(starts[-1] + q)
    return SimpleNamespace(q_start=starts, ctx_before=list(before), **kw)


def test_long_or_uneven_decode_batches_are_marked():
    assert not attn.deal_tiles_hint([20000])                        # one request: more splits instead
    assert attn.deal_tiles_hint([20000, 100])                       # beyond the long-context mark
    assert attn.deal_tiles_hint([9000] * 8)
    assert attn.deal_tiles_hint([4096] + [500] * 31)                # one request much longer than the mean
    assert not attn.deal_tiles_hint([4096] * 32)                    # long-ish but even
    assert not attn.deal_tiles_hint([1500] + [10] * 7)              # uneven but short
    assert not attn.deal_tiles_hint([1040] * 8)


@pytest.fixture(autouse=True)
def a_gpu_of_148_multiprocessors(monkeypatch):
    """The policies ask the device for its size; without one, these tests state the B200's."""
    monkeypatch.setattr(attn, "SM_COUNT", 148)


def test_which_decode_kernel_takes_a_step():
    plain_step, dealt = False, True
    assert not attn.decode_lean_preferred(8, 8, 128, plain_step)    # 64 pairs: a block (or four) each
    assert not attn.decode_lean_preferred(37, 8, 128, plain_step)   # 296 pairs still fit at once
    assert attn.decode_lean_preferred(38, 8, 128, plain_step)
    assert attn.decode_lean_preferred(8, 8, 128, dealt) and not attn.decode_lean_preferred(1, 8, 128, dealt)
    assert not attn.decode_lean_preferred(18, 8, 256, plain_step) and attn.decode_lean_preferred(18, 8, 256, dealt)
    assert attn.decode_lean_preferred(19, 8, 256, plain_step)       # one block per SM at head size 256: 152 pairs > 148
    assert not attn.decode_lean_preferred(5000, 8, 128, dealt)      # the kernel's schedule holds 4096 requests
    assert attn.decode_splits(8, 8) == 4 and attn.decode_splits(1, 8) == 32 and attn.decode_splits(64, 8) == 1
    # clusters of up to 8 splits, of more than 4 only while they leave room; steps of the long-context kind up to 32
    assert [attn.decode_tma_splits(r, 8, False) for r in (1, 2, 4, 8, 16, 32, 64)] == [8, 8, 6, 4, 2, 1, 1]
    assert [attn.decode_tma_splits(r, 8, True) for r in (1, 2, 4, 8)] == [32, 18, 9, 4]
    # what a recorded decode step is keyed by: (tiles dealt out, long context)
    assert attn.decode_step_kind([1040] * 8) == (False, False) and attn.decode_step_kind([20000]) == (False, True)
    assert attn.decode_step_kind([20000, 100]) == (True, False) and attn.decode_step_kind([]) == (False, False)


def test_decoding_requests_of_a_mixed_step():
    assert not attn.mixed_step_splits_off_decodes(host([1, 1, 2047], [100, 900, 0]))
    assert attn.mixed_step_splits_off_decodes(host([1, 1, 2047], [3000, 2000, 0]))
    assert not attn.mixed_step_splits_off_decodes(host([2047, 2], [9000, 9000]))      # nobody brings one token
    assert not attn.mixed_step_splits_off_decodes(SimpleNamespace(q_start=[0, 1], ctx_before=[]))


@pytest.mark.parametrize("per, q_lens, before, good", [
    # (heads per KV head, tokens, cached before, shares of the longest tile among the measured options within 10 % of the best)
    (3, [1, 2047], [14012, 816], {4, 6, 8}),                # 465 us whole; 174 / 175 / 181 us
    (3, [1, 2047], [12596, 3830], {2, 4, 6, 8}),            # 481; 291 / 283 / 295 / 297
    (3, [1, 1545, 502], [2332, 7908, 0], {1}),              # 264; divided 289 and more
    (3, [2048], [12000], {2, 3}),                           # 392 blocks: 587; 512 / 512
    (3, [2048], [6000], {2, 3}),                            # 323; 300 / 312
    (3, [2048], [3000], {1, 2}),                            # 196 / 193
    (3, [512], [3584], {2}),                                # 128 blocks: 89; 73
    (3, [2048], [0], {1}),                                  # 70; 82
    (4, [1, 2047], [14012, 816], {3, 4, 6, 8}),             # 451; 207 / 200 / 208 / 209
    (4, [1, 2047], [12596, 3830], {2, 3, 4}),               # 419; 306 / 330 / 327
    (4, [2048], [12000], {1}),                              # 512 blocks: 583; divided 607 and more
    (4, [2048], [6000], {1}),
    (4, [512], [3584], {2}),                                # 87; 72
    (4, [2048], [0], {1}),
    (4, [8192], [0], {1}),
])
def test_key_splits_of_prompt_tiles_against_measured_steps(per, q_lens, before, good):
    splits, limit = attn.prefill_kv_splits(host(q_lens, before), per, 8, 128)
    longest = max(b + q - 1 for q, b in zip(q_lens, before)) // 64 + 1
    assert splits in good, (splits, limit)
    if splits > 1:
        assert limit >= attn.PREFILL_SPLIT_MIN_TILES and splits == -(-longest // limit)


def test_key_splits_ignore_what_another_kernel_takes():
    step = host([1, 2047], [14012, 816])
    assert attn.prefill_kv_splits(step, 3, 8, 128)[0] > 1
    assert attn.prefill_kv_splits(step, 3, 8, 128, skip_single=True) == (1, 1)        # the long request is not the prompt kernel's
    assert attn.prefill_kv_splits(host([1, 1], [9000, 9000]), 3, 8, 128, skip_single=True) == (1, 1)
    assert attn.prefill_kv_splits(SimpleNamespace(q_start=[0, 8], ctx_before=[]), 4, 8, 128) == (1, 1)


def test_model_of_the_prompt_kernels_launch():
    items = [(100, 1.0)] * 37
    one_round = attn._prefill_step_length(items, 37, 1, 1)
    assert one_round == 100 + attn.PREFILL_SPLIT_START_UP
    assert attn._prefill_step_length(items + [(100, 1.0)], 37, 1, 1) == 2 * one_round             # a 38th block waits
    halves = attn._prefill_step_length(items + [(100, 1.0)], 37, 2, 50)
    assert one_round < halves < 2 * one_round                                                     # 76 halves: three short rounds
    assert attn._prefill_step_length([(300, 1.4)] + [(10, 1.0)] * 30, 37, 1, 1) == 300 * 1.4 + attn.PREFILL_SPLIT_START_UP
