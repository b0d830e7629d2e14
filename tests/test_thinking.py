"""The thinking-budget control (host side of the sampling path), checked with
the reference's own deterministic cases: every test below replays one of
tests/unit/thinking.rs of the reference (same toy vocabulary: one id per
character from 10 000 up, the markers 1..4; same texts), through the C ABI."""
import random

import pytest


@pytest.fixture(scope="module")
def T(lily):
    import lily_b200.thinking as t
    return t


THINK_END, TOOL_CALL, TOOL_CALL_END, IM_END, CHAR = 1, 2, 3, 4, 10_000


def is_added(i):
    return i <= IM_END


def encode(text):
    return [CHAR + ord(c) for c in text]


def text(ids):
    names = {THINK_END: "</think>", TOOL_CALL: "<tool_call>", TOOL_CALL_END: "</tool_call>",
             IM_END: "<|im_end|>"}
    return "".join(names.get(i) or chr(i - CHAR) for i in ids)


def text_ids(t):
    ids, rest = [], t
    while rest:
        if rest.startswith("</think>"):
            ids.append(THINK_END)
            rest = rest[len("</think>"):]
        else:
            ids.append(CHAR + ord(rest[0]))
            rest = rest[1:]
    return ids


def texts(T):
    return T.ThinkingTexts(["Act now.", "Go."],
                           [T.NudgeLevel(0.5, ["Half.", "Halfway."]),
                            T.NudgeLevel(0.75, ["Three quarters."])])


def tokens(T, tx=None):
    return T.ThinkingTokens(THINK_END, TOOL_CALL, TOOL_CALL_END, tx if tx is not None else texts(T),
                            encode, is_added)


def control(T, settings, opens=True, tk=None):
    tk = tk or tokens(T)
    c = T.ThinkingControl(tk, settings, opens)
    c._keep = tk
    return c


def word(c, t):
    return c.decide(100, t)


def budget(T, n, grace, **kw):
    return T.ThinkingSettings(budget=n, grace=grace, **kw)


def after(T, a):
    assert a.kind == T.AFTER, a
    return a.ids


def test_nothing_happens_without_an_open_block_or_after_it_closed(T):
    s = budget(T, 2, 0, tool_call_ends_thinking=True)
    closed = control(T, s, opens=False)
    assert not closed.may_act_next()
    for _ in range(10):
        assert word(closed, "x\n") == T.Keep
    assert closed.decide(TOOL_CALL, "<tool_call>") == T.Keep
    assert closed.decide_stop() == T.Keep
    assert closed.closed() is None
    c = control(T, s)
    assert c.decide(THINK_END, "</think>") == T.Keep
    assert not c.is_open() and not c.may_act_next()
    for _ in range(10):
        assert word(c, "x\n") == T.Keep
    assert c.decide(TOOL_CALL, "<tool_call>") == T.Keep
    assert c.decide_stop() == T.Keep
    assert c.closed() is None


def test_a_tool_call_at_a_line_start_ends_thinking_with_only_the_close_tag(T):
    on = T.ThinkingSettings(tool_call_ends_thinking=True)
    c = control(T, on)
    assert c.may_act_next()
    a = c.decide(TOOL_CALL, "<tool_call>")
    assert a.kind == T.BEFORE and text(a.ids) == "</think>\n\n"
    assert not c.is_open()
    assert c.closed() == T.Closed(T.CLOSED_TOOL_CALL, 0)
    c = control(T, on)
    assert word(c, "Let me look") == T.Keep
    assert not c.may_act_next()
    assert word(c, ".\n") == T.Keep
    assert c.may_act_next()
    assert c.decide(TOOL_CALL, "<tool_call>").kind == T.BEFORE
    assert c.closed().thinking_tokens == 2
    c = control(T, on)
    assert word(c, "I would call ") == T.Keep
    assert c.decide(TOOL_CALL, "<tool_call>") == T.Keep
    assert c.is_open()
    c = control(T, T.ThinkingSettings())
    assert not c.may_act_next()
    assert c.decide(TOOL_CALL, "<tool_call>") == T.Keep
    assert c.is_open()


def test_the_budget_closes_at_the_first_line_end_from_the_budget_on(T):
    c = control(T, budget(T, 5, 4))
    for t in "abc":
        assert word(c, t) == T.Keep
        assert c.may_act_next()
    assert word(c, "d") == T.Keep
    assert word(c, "e") == T.Keep
    assert word(c, " f") == T.Keep
    assert text(after(T, word(c, "g\n"))) == "Act now.\n</think>\n\n"
    assert c.closed() == T.Closed(T.CLOSED_BUDGET, 7)
    assert not c.is_open() and not c.may_act_next()


def test_the_close_puts_its_preface_on_a_line_of_its_own_at_a_clean_seam(T):
    def close(last):
        c = control(T, budget(T, 1, 0))
        return text(after(T, word(c, last)))
    assert close("x\n\n") == "Act now.\n</think>\n\n"
    assert close("x\n") == "Act now.\n</think>\n\n"
    assert close("x") == "\n\nAct now.\n</think>\n\n"
    assert close("7") == "\n\nAct now.\n</think>\n\n"
    assert close("é") == "\n\nAct now.\n</think>\n\n"
    assert close("x.") == " \n\nAct now.\n</think>\n\n"
    assert close("**") == " \n\nAct now.\n</think>\n\n"
    c = control(T, budget(T, 1, 0))
    assert word(c, "x ") == T.Keep
    assert word(c, "\t") == T.Keep
    assert c.is_open() and c.may_act_next()
    assert text(after(T, word(c, "y"))) == "\n\nAct now.\n</think>\n\n"


def test_grace_waits_for_a_line_then_a_sentence_then_forces(T):
    c = control(T, budget(T, 2, 0))
    assert word(c, "a") == T.Keep
    assert word(c, "b").kind == T.AFTER
    c = control(T, budget(T, 2, 3))
    assert word(c, "a") == T.Keep
    assert word(c, "b.") == T.Keep
    assert word(c, " c.") == T.Keep
    assert word(c, " d.") == T.Keep
    assert text(after(T, word(c, " e."))).startswith(" \n\n")
    c = control(T, budget(T, 1, 2))
    for _ in range(4):
        assert word(c, "w") == T.Keep
    assert word(c, "w").kind == T.AFTER


def test_nothing_lands_inside_a_code_fence_or_a_tool_call(T):
    c = control(T, budget(T, 3, 10))
    assert word(c, "```rust\n") == T.Keep
    for _ in range(5):
        assert word(c, "let x = 1;\n") == T.Keep
    assert word(c, "```") == T.Keep
    assert word(c, "\n").kind == T.AFTER
    c = control(T, budget(T, 1, 10))
    assert word(c, "  ``") == T.Keep
    assert word(c, "`\n") == T.Keep
    assert word(c, "x\n") == T.Keep
    c = control(T, budget(T, 1, 2))
    assert word(c, "```\n") == T.Keep
    for _ in range(50):
        assert word(c, "code\n") == T.Keep
    assert c.is_open() and c.may_act_next()
    assert word(c, "```").kind == T.AFTER
    c = control(T, budget(T, 2, 0))
    assert word(c, "```\n") == T.Keep
    assert word(c, "x") == T.Keep
    assert word(c, "\n") == T.Keep
    c = control(T, budget(T, 2, 1))
    assert c.decide(TOOL_CALL, "<tool_call>") == T.Keep
    for _ in range(20):
        assert word(c, "<parameter=x>\n") == T.Keep
    assert c.decide(TOOL_CALL_END, "</tool_call>").kind == T.AFTER
    c = control(T, budget(T, 2, 10))
    assert c.decide(TOOL_CALL, "<tool_call>") == T.Keep
    assert word(c, "<function=f>\n") == T.Keep
    assert c.decide(TOOL_CALL_END, "</tool_call>") == T.Keep
    assert word(c, "\n").kind == T.AFTER


def test_nudges_come_at_their_fractions_and_the_block_stays_open(T):
    c = control(T, budget(T, 20, 4, nudges=True))
    inserted = []
    for i in range(1, 20):
        a = word(c, "b\n" if i % 2 == 0 else "a")
        if a.kind == T.AFTER:
            inserted.append((c.thinking_tokens(), text(a.ids)))
        else:
            assert a == T.Keep
    assert inserted == [(10, "Half.\n\n"), (16, "Three quarters.\n\n")]
    assert c.is_open() and c.nudged() == 2 and c.closed() is None
    assert word(c, "end\n").kind == T.AFTER
    assert c.closed().by == T.CLOSED_BUDGET
    c = control(T, budget(T, 20, 4))
    for _ in range(19):
        assert word(c, "x\n") == T.Keep
    c = control(T, T.ThinkingSettings(nudges=True))
    for _ in range(100):
        assert word(c, "x\n") == T.Keep


def test_nudge_variants_rotate_with_the_seed(T):
    def first_nudge(seed):
        c = control(T, budget(T, 4, 0, nudges=True, seed=seed))
        assert word(c, "x") == T.Keep
        return text(after(T, word(c, "y\n")))
    assert first_nudge(0) == "Half.\n\n"
    assert first_nudge(1) == "Halfway.\n\n"
    assert first_nudge(2) == "Half.\n\n"
    assert first_nudge(2**64 - 1) == "Halfway.\n\n"

    def close(seed):
        c = control(T, budget(T, 1, 0, seed=seed))
        return text(after(T, word(c, "x\n\n")))
    assert close(0) == "Act now.\n</think>\n\n"
    assert close(1) == "Go.\n</think>\n\n"
    assert close(2**64 - 1) == "Go.\n</think>\n\n"
    c = control(T, budget(T, 4, 0, nudges=True, seed=2**64 - 1))
    assert word(c, "x") == T.Keep
    assert word(c, "y\n").kind == T.AFTER
    assert text(after(T, word(c, "z\n"))) == "Three quarters.\n\n"


def test_a_nudge_lands_only_at_a_line_end_within_its_window(T):
    c = control(T, budget(T, 20, 2, nudges=True))
    for _ in range(9):
        assert word(c, "w") == T.Keep
    for _ in range(3):
        assert word(c, " end.") == T.Keep
    assert word(c, "\n") == T.Keep
    assert c.nudged() == 0
    assert word(c, "a") == T.Keep
    assert word(c, "b") == T.Keep
    assert text(after(T, word(c, "c\n"))) == "Three quarters.\n\n"
    assert c.nudged() == 1


def test_a_tool_call_in_a_fence_or_inside_a_kept_call_does_not_end_thinking(T):
    on = T.ThinkingSettings(tool_call_ends_thinking=True)
    c = control(T, on)
    assert word(c, "```xml\n") == T.Keep
    assert not c.may_act_next()
    assert c.decide(TOOL_CALL, "<tool_call>") == T.Keep
    assert c.decide(TOOL_CALL_END, "</tool_call>") == T.Keep
    assert word(c, "\n```\n") == T.Keep
    assert c.is_open() and c.may_act_next()
    assert c.decide(TOOL_CALL, "<tool_call>").kind == T.BEFORE
    c = control(T, on)
    assert word(c, "Like ") == T.Keep
    assert c.decide(TOOL_CALL, "<tool_call>") == T.Keep
    assert c.is_open()
    assert word(c, " does.\n") == T.Keep
    assert c.may_act_next()
    assert c.decide(TOOL_CALL, "<tool_call>").kind == T.BEFORE


def quoted_call_then_real_one(T, fenced, closing):
    on = T.ThinkingSettings(tool_call_ends_thinking=True)
    c = control(T, on)
    for line in fenced:
        assert word(c, line) == T.Keep
        assert not c.may_act_next(), (fenced, line)
    assert c.decide(TOOL_CALL, "<tool_call>") == T.Keep
    assert word(c, "\n") == T.Keep
    assert word(c, closing) == T.Keep
    assert c.may_act_next(), (fenced, closing)
    assert c.decide(TOOL_CALL, "<tool_call>").kind == T.BEFORE


def test_fences_open_and_close_as_commonmark_has_them(T):
    quoted_call_then_real_one(T, ["```\n"], "```\n")
    quoted_call_then_real_one(T, ["````md\n", "```\n", "text\n"], "````\n")
    quoted_call_then_real_one(T, ["```\n"], "   `````  \n")
    quoted_call_then_real_one(T, ["~~~ text\n", "```\n", "~~\n"], "~~~~\n")
    quoted_call_then_real_one(T, ["```\n", "```rust\n"], "```\n")
    quoted_call_then_real_one(T, ["~~~\n", "~~~ \n"], "~~~\t\r\n")
    on = T.ThinkingSettings(tool_call_ends_thinking=True)
    for line in ["    ```\n", "``\n", "``` a`b\n", "\t```\n"]:
        c = control(T, on)
        assert word(c, line) == T.Keep
        assert c.decide(TOOL_CALL, "<tool_call>").kind == T.BEFORE, line
    c = control(T, budget(T, 1, 0))
    assert word(c, "~~~~\n") == T.Keep
    assert word(c, "~~~\n") == T.Keep
    assert word(c, "~~~~") == T.Action(T.AFTER, text_ids(" \n\nAct now.\n</think>\n\n"))
    c = control(T, budget(T, 1, 0))
    assert word(c, "```") == T.Keep
    assert word(c, "py") == T.Keep
    assert word(c, "\n") == T.Keep


def test_only_a_call_at_a_line_start_outside_a_fence_holds_the_close_back(T):
    c = control(T, budget(T, 1, 4))
    assert word(c, "Use ") == T.Keep
    assert c.decide(TOOL_CALL, "<tool_call>") == T.Keep
    assert word(c, " here.\n").kind == T.AFTER
    c = control(T, budget(T, 1, 4))
    assert word(c, "```\n") == T.Keep
    assert c.decide(TOOL_CALL, "<tool_call>") == T.Keep
    assert word(c, "\n") == T.Keep
    assert word(c, "```\n").kind == T.AFTER
    c = control(T, budget(T, 1, 4))
    assert c.decide(TOOL_CALL, "<tool_call>") == T.Keep
    assert word(c, "\n<parameter=x>\n```\n") == T.Keep
    assert c.decide(TOOL_CALL_END, "</tool_call>") == T.Keep
    assert word(c, "\n").kind == T.AFTER


def test_a_nudge_that_cannot_leave_a_fence_is_dropped(T):
    c = control(T, budget(T, 40, 2, nudges=True))
    assert word(c, "```\n") == T.Keep
    for _ in range(36):
        assert word(c, "code\n") == T.Keep
    assert c.nudged() == 0
    assert word(c, "```\n") == T.Keep
    assert c.nudged() == 0


def test_the_control_never_acts_unannounced(T):
    pieces = ["a", "b.", " c", "\n", "\n\n", "x\n", "```", "``", "`\n", "  ", "end.", "?", "~~~",
              "````\n", " "]
    rng = random.Random(7)
    tk = tokens(T)
    for trial in range(400):
        s = T.ThinkingSettings(budget=rng.randrange(1, 60) if rng.random() < 0.8 else None,
                               grace=rng.randrange(0, 6), nudges=rng.random() < 0.5,
                               tool_call_ends_thinking=rng.random() < 0.5,
                               seed=rng.getrandbits(64))
        c = control(T, s, tk=tk)
        for step in range(120):
            announced = c.may_act_next()
            r = rng.randrange(100)
            if r < 2:
                a = c.decide_stop()
            elif r < 4:
                a = c.decide(TOOL_CALL, "<tool_call>")
            elif r < 8:
                a = c.decide(TOOL_CALL_END, "</tool_call>")
            elif r < 9:
                a = c.decide(THINK_END, "</think>")
            else:
                a = word(c, rng.choice(pieces))
            assert a == T.Keep or announced, (trial, step, a, s)


def test_texts_validate_and_read_from_json(T):
    T.ThinkingTokens(1, 2, 3, None, encode, is_added)  # the built-in texts
    bad_order = T.ThinkingTexts([], [T.NudgeLevel(0.75, ["a"]), T.NudgeLevel(0.5, ["b"])])
    with pytest.raises(ValueError):
        T.ThinkingTokens(1, 2, 3, bad_order, encode, is_added)
    with pytest.raises(ValueError):
        T.ThinkingTokens(1, 2, 3, T.ThinkingTexts([], [T.NudgeLevel(1.0, ["a"])]), encode, is_added)
    spelled = T.ThinkingTexts(["</think>"], [])
    marker = lambda t: [THINK_END] if "</think>" in t else encode(t)
    with pytest.raises(ValueError):
        T.ThinkingTokens(1, 2, 3, spelled, marker, is_added)
    im_end = lambda t: [IM_END] if "<|im_end|>" in t else encode(t)
    ending = T.ThinkingTexts([], [T.NudgeLevel(0.5, ["Done<|im_end|>"])])
    with pytest.raises(ValueError) as e:
        T.ThinkingTokens(1, 2, 3, ending, im_end, is_added)
    assert "added token" in str(e.value)
    bare = T.ThinkingTokens(1, 2, 3, T.ThinkingTexts([], []), encode, is_added)
    c = T.ThinkingControl(bare, budget(T, 1, 0), True)
    assert text(after(T, word(c, "x"))) == "\n</think>\n\n"
    c = T.ThinkingControl(bare, budget(T, 1, 0), True)
    assert text(after(T, word(c, "x\n"))) == "</think>\n\n"
    js = '{"close": ["Stop."], "nudges": [{"at": 0.6, "texts": ["Soon."]}]}'
    parsed = T.ThinkingTokens(1, 2, 3, None, encode, is_added, json_text=js)
    c = T.ThinkingControl(parsed, budget(T, 10, 0, nudges=True), True)
    for _ in range(5):
        assert word(c, "x") == T.Keep
    assert text(after(T, word(c, "y\n"))) == "Soon.\n\n"  # 0.6 * 10 = 6
    for _ in range(3):
        assert word(c, "x\n") == T.Keep
    assert text(after(T, word(c, "x\n"))) == "Stop.\n</think>\n\n"
    with pytest.raises(ValueError):
        T.ThinkingTokens(1, 2, 3, None, encode, is_added, json_text='{"closes": []}')
    with pytest.raises(ValueError):
        T.ThinkingTokens(1, 2, 3, None, encode, is_added,
                         json_text='{"nudges": [{"at": 0.5, "texts": ["a"], "x": 1}]}')


def test_only_a_prompt_ending_in_an_open_block_opens_thinking(T):
    assert T.opens_thinking("<|im_start|>assistant\n<think>\n")
    assert not T.opens_thinking("<|im_start|>assistant\n<think>\n\n</think>\n\n")
    assert not T.opens_thinking("<|im_start|>assistant\n")


def test_an_end_of_turn_inside_the_block_is_replaced_once_with_a_budget(T):
    def replaced(last):
        c = control(T, budget(T, 1000, 4))
        assert word(c, last) == T.Keep
        assert c.may_act_next()
        a = c.decide_stop()
        assert a.kind == T.REPLACE
        assert not c.is_open()
        assert c.closed() == T.Closed(T.CLOSED_END_OF_TURN, 1)
        assert c.decide_stop() == T.Keep
        assert not c.may_act_next()
        return text(a.ids)
    assert replaced("Let me write the code now.\n") == "</think>\n\n"
    assert replaced("Let me write the code now.") == " \n</think>\n\n"
    assert replaced("Let me write the code") == "\n</think>\n\n"
    assert replaced("Let me write ") == "\n</think>\n\n"
    assert replaced("```\n") == "</think>\n\n"
    c = control(T, budget(T, 10, 0))
    assert c.decide_stop() == T.Action(T.REPLACE, text_ids("</think>\n\n"))
    assert c.closed().thinking_tokens == 0
    c = control(T, T.ThinkingSettings(tool_call_ends_thinking=True))
    assert word(c, "done") == T.Keep
    assert c.decide_stop() == T.Keep
    assert not c.may_act_next()
    c = control(T, budget(T, 1, 0))
    assert word(c, "x\n").kind == T.AFTER
    assert c.decide_stop() == T.Keep
    assert c.closed().by == T.CLOSED_BUDGET


def test_the_models_own_close_at_a_threshold_or_during_a_wait_wins(T):
    c = control(T, budget(T, 3, 4))
    assert word(c, "a") == T.Keep
    assert word(c, "b") == T.Keep
    assert c.may_act_next()
    assert c.decide(THINK_END, "</think>") == T.Keep
    assert not c.is_open()
    assert (c.closed(), c.thinking_tokens()) == (None, 2)
    assert word(c, "\n") == T.Keep
    c = control(T, budget(T, 1, 4))
    assert word(c, "a") == T.Keep
    assert c.decide(THINK_END, "</think>") == T.Keep
    assert word(c, "\n\n") == T.Keep
    assert c.closed() is None
    for waited in (0, 2):
        c = control(T, budget(T, 20, 4, nudges=True))
        for _ in range(9 + waited):
            assert word(c, "w") == T.Keep
        assert c.decide(THINK_END, "</think>") == T.Keep
        assert word(c, "\n") == T.Keep
        assert (c.nudged(), c.closed()) == (0, None)


def test_a_close_cut_short_is_not_reported_as_emitted(T):
    c = control(T, budget(T, 1, 0))
    assert not c.close_emitted([])
    ids = after(T, word(c, "x\n"))
    generated = [100] + ids
    assert c.close_emitted(generated)
    cut = ids.index(THINK_END)
    assert not c.close_emitted(generated[:1 + cut])
    assert not c.close_emitted([100])


def test_settings_any(T):
    # src/thinking.rs:349-351
    assert not T.ThinkingSettings().any()
    assert T.ThinkingSettings(budget=5).any()
    assert T.ThinkingSettings(tool_call_ends_thinking=True).any()
    assert not T.ThinkingSettings(nudges=True).any()


# ---- src/generate.rs:121-169, cases of tests/unit/generate.rs ----------------

def recorder(stop_at=None):
    seen = []

    def cb(t):
        seen.append(t)
        return t != stop_at
    return seen, cb


def test_an_inserted_group_is_emitted_whole_even_when_the_callback_stops(T):
    seen, cb = recorder()
    toks = [1, 2]
    assert T.emit_acted(T.Action(T.BEFORE, [7, 8]), 9, toks, 100, cb) is None
    assert toks == [1, 2, 7, 8, 9] and seen == [7, 8, 9]
    seen, cb = recorder(9)
    toks = [1]
    assert T.emit_acted(T.Action(T.AFTER, [7, 8]), 9, toks, 100, cb) == T.FINISH_CALLBACK
    assert toks == [1, 9, 7, 8] and seen == [9, 7, 8]
    _, cb = recorder(7)
    toks = []
    assert T.push_group(toks, [7, 8, 9], 100, cb) == T.FINISH_CALLBACK
    assert toks == [7, 8, 9]
    with pytest.raises(ValueError):
        T.emit_acted(T.Keep, 9, [], 100, cb)


def test_only_the_length_cuts_an_inserted_group_short(T):
    seen, cb = recorder()
    toks = [1, 2]
    assert T.emit_acted(T.Action(T.AFTER, [7, 8, 9]), 5, toks, 4, cb) == T.FINISH_LENGTH
    assert toks == [1, 2, 5, 7] and seen == [5, 7]
    _, cb = recorder()
    toks = [1]
    assert T.push_group(toks, [7, 8], 3, cb) == T.FINISH_LENGTH
    assert toks == [1, 7, 8]
    _, cb = recorder()
    toks = [1]
    assert T.emit_acted(T.Action(T.BEFORE, [7, 8]), 9, toks, 3, cb) == T.FINISH_LENGTH
    assert toks == [1, 7, 8]


def test_a_replaced_stop_token_is_dropped_and_the_close_emitted_in_its_place(T):
    seen, cb = recorder()
    toks = [1, 2]
    assert T.emit_acted(T.Action(T.REPLACE, [7, 8]), 99, toks, 100, cb) is None
    assert toks == [1, 2, 7, 8] and seen == [7, 8]
    seen, cb = recorder()
    toks = [1, 2]
    assert T.emit_acted(T.Action(T.REPLACE, [7, 8, 9]), 99, toks, 4, cb) == T.FINISH_LENGTH
    assert toks == [1, 2, 7, 8] and seen == [7, 8]
    seen, cb = recorder(7)
    toks = [1]
    assert T.emit_acted(T.Action(T.REPLACE, [7, 8]), 99, toks, 100, cb) == T.FINISH_CALLBACK
    assert toks == [1, 7, 8] and seen == [7, 8]


def test_every_insertion_stops_exactly_at_max_tokens(T):
    groups = [(T.BEFORE, [7, 8, 9]), (T.AFTER, [9, 7, 8]), (T.REPLACE, [7, 8])]
    for kind, whole in groups:
        for room in range(len(whole) + 2):
            seen, cb = recorder()
            toks = [1]
            mx = 1 + room
            end = T.emit_acted(T.Action(kind, [7, 8]), 9, toks, mx, cb)
            fits = min(room, len(whole))
            if kind == T.AFTER:
                fits = max(fits, 1)
            assert toks[1:] == whole[:fits], (kind, room)
            assert seen == whole[:fits], (kind, room)
            assert end == (T.FINISH_LENGTH if len(toks) >= mx else None), (kind, room)
