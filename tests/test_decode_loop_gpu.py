"""A decode loop that joins the thinking control to the sampling kernel.

The reference's contract (src/generate.rs:76-82, 892-907; src/kernels/metal/
sample.metal:509-511): a draw is keyed by (seed, index), the index being the
token's place in the generation, inserted tokens included, so an insertion of n
tokens skips n indices of the seed's stream; and only tokens the sampler DREW
enter the penalty counts, because inserted tokens never pass through it.

Here the tokens the control inserts (lily_thinking_decide, emitted in the order
lily_emit_acted gives) go through the kernel's `forced_ids`: a row with a
pending token returns it without drawing and without counting. The GPU loop
(two rows in one batch: one under a thinking budget, one plain) has to produce
the token sequences and the histogram slots of a CPU loop built from the
oracle, a second control of the same settings and plain Python lists.
"""
import numpy as np
import pytest

import oracle
from gpu_util import np_u32

pytestmark = pytest.mark.gpu

THINK_END, TOOL_CALL, TOOL_CALL_END, IM_END, CHAR = 1, 2, 3, 4, 10_000
VOCAB = 10_240
LETTERS = "abcdefgh \n"
SEEDS = (71, 72)
PARAMS = dict(temperature=0.9, top_k=8, top_p=0.95, repetition_penalty=1.3, presence_penalty=0.4,
              frequency_penalty=0.2)
N_TOKENS = 48


def encode(text):
    return [CHAR + ord(c) for c in text]


def text_of(token):
    names = {THINK_END: "</think>", TOOL_CALL: "<tool_call>", TOOL_CALL_END: "</tool_call>",
             IM_END: "<|im_end|>"}
    return names.get(token) or chr(token - CHAR)


def model_logits(row, index):
    """The stand-in for the model: seeded logits for (row, place in the generation);
    a handful of characters (a line end among them) carry nearly all the mass."""
    rng = np.random.default_rng([9001, row, index])
    x = rng.standard_normal(VOCAB, dtype=np.float32) - np.float32(12.0)
    for c in LETTERS:
        x[CHAR + ord(c)] = np.float32(2.0) + rng.standard_normal(dtype=np.float32)
    return x


def make_control(T):
    texts = T.ThinkingTexts(["Act now.", "Go."],
                            [T.NudgeLevel(0.5, ["Half.", "Halfway."]), T.NudgeLevel(0.75, ["Three quarters."])])
    tokens = T.ThinkingTokens(THINK_END, TOOL_CALL, TOOL_CALL_END, texts, encode, lambda i: i <= IM_END)
    control = T.ThinkingControl(tokens, T.ThinkingSettings(budget=10, grace=6, nudges=True, seed=SEEDS[0]),
                                True)
    control._keep = tokens
    return control


def emitted(T, control, drawn):
    """What a draw puts into the generation: itself, or the control's group around it."""
    action = control.decide(drawn, text_of(drawn))
    if action.kind == T.KEEP:
        return [drawn], False
    out = []
    T.emit_acted(action, drawn, out, 1 << 30, lambda t: True)
    return out, True


def cpu_loop(T):
    control = make_control(T)
    tokens = [[], []]
    counts = [np.zeros(VOCAB, dtype=np.uint32) for _ in range(2)]
    draws = [0, 0]
    inserted = 0
    for row in range(2):
        p = oracle.params(**PARAMS, seed=SEEDS[row])
        while len(tokens[row]) < N_TOKENS:
            index = len(tokens[row])
            d = oracle.sample(model_logits(row, index), p, float(oracle.uniform_for(SEEDS[row], index)),
                              counts=counts[row])
            assert d.status == oracle.OK
            counts[row][d.token] += 1  # the draw is counted; nothing else ever is
            draws[row] += 1
            if row == 0:
                group, acted = emitted(T, control, int(d.token))
                inserted += len(group) - 1
                tokens[row].extend(group)
            else:
                tokens[row].append(int(d.token))
    return tokens, counts, draws, inserted


def test_inserted_tokens_skip_draw_indices_and_stay_out_of_the_counts(cuda, lily):
    import lily_b200.thinking as T

    torch = cuda
    want_tokens, want_counts, want_draws, inserted = cpu_loop(T)
    assert inserted > 0, "the scenario must make the control insert something"

    control = make_control(T)
    scratch = lily.SamplerScratch(VOCAB, max_rows=2, counts_table=True)
    params = [lily.SamplingParams(**PARAMS, seed=SEEDS[row]) for row in range(2)]
    tokens = [[], []]
    pending = []            # row 0: tokens on their way into the generation through forced_ids
    forced_steps = 0
    out = torch.zeros(2, dtype=torch.int32, device="cuda")
    status = torch.zeros(2, dtype=torch.int32, device="cuda")
    done = lambda row: len(tokens[row]) >= N_TOKENS and not (row == 0 and pending)
    while not (done(0) and done(1)):
        index = [len(tokens[0]), len(tokens[1])]
        logits = torch.from_numpy(np.stack([model_logits(r, index[r]) for r in range(2)])).cuda()
        # A finished row is parked on a forced id: it neither draws nor counts.
        forced = np.array([pending[0] if pending else (IM_END if done(0) else -1),
                           IM_END if done(1) else -1], dtype=np.int32)
        was_done = [done(0), done(1)]
        scratch.sample_batch(logits, params, out, steps=index, count_slots=[0, 1],
                             forced_ids=torch.from_numpy(forced).cuda(), out_status=status)
        torch.cuda.synchronize()
        got, st = np_u32(out), np_u32(status)
        if pending:
            assert st[0] == lily.ROW_FORCED and got[0] == pending[0]
            tokens[0].append(pending.pop(0))
            forced_steps += 1
        elif not was_done[0]:
            assert st[0] == lily.ROW_OK
            group, acted = emitted(T, control, int(got[0]))
            if acted:
                pending = group  # the group, with the draw at its place, goes in token by token
            else:
                tokens[0].append(int(got[0]))
        if not was_done[1]:
            assert st[1] == lily.ROW_OK
            tokens[1].append(int(got[1]))
    assert scratch.status() == lily.OK
    assert tokens[0] == want_tokens[0], "the row under the thinking control"
    assert tokens[1] == want_tokens[1], "the plain row"
    assert forced_steps > 0
    # The histogram slots hold the draws and only the draws.
    for slot in range(2):
        got_counts = scratch.read_counts(slot)
        assert np.array_equal(got_counts, want_counts[slot]), f"slot {slot}"
        assert int(got_counts.sum()) == want_draws[slot]
    assert want_draws[0] == len(tokens[0]) - inserted and want_draws[1] == len(tokens[1])
    scratch.close()
