"""The request -> parameters layer against the reference's own cases
(tests/unit/serve.rs:160-178 sampling_defaults_apply_overrides;
tests/unit/serve/api.rs:131-248 thinking budgets, defaults and fields;
src/serve/api.rs:798-834 resolve_sampling). Host logic only: no GPU."""
import json

import pytest


@pytest.fixture(scope="module")
def rq(lily):
    import lily_b200.request as request

    return request


def test_sampling_defaults_apply_overrides(lily, rq):
    # tests/unit/serve.rs:160-178
    cfg = b'{"do_sample": true, "temperature": 1.0, "top_k": 20, "top_p": 0.95}'
    base = rq.sampling_defaults(cfg)
    assert (base.temperature, base.top_k, round(base.top_p, 6)) == (1.0, 20, 0.95)
    over = rq.sampling_defaults(cfg, rq.Overrides(present=rq.HAS_TEMPERATURE, temperature=0.0))
    assert over.is_greedy()
    # No file: OpenAI's defaults (src/serve.rs:1776-1785).
    d = rq.sampling_defaults(None)
    assert (d.temperature, d.top_k, d.top_p, d.min_p, d.repetition_penalty) == (1.0, 0, 1.0, 0.0, 1.0)
    # do_sample false is greedy unless a temperature is given as well (file order).
    assert rq.sampling_defaults(b'{"do_sample": false}').temperature == 0.0
    assert rq.sampling_defaults(b'{"do_sample": false, "temperature": 0.5}').temperature == 0.5
    # The file has no frequency_penalty member (src/serve.rs:1788-1811).
    assert rq.sampling_defaults(b'{"frequency_penalty": 1.5, "presence_penalty": 0.25}').frequency_penalty == 0.0
    assert rq.sampling_defaults(b'{"presence_penalty": 0.25}').presence_penalty == 0.25
    # Validation is the last step; the unvalidated read keeps what it read.
    with pytest.raises(lily.LilyError):
        rq.sampling_defaults(b'{"top_p": 1.5}')
    assert rq.sampling_defaults(b'{"top_p": 1.5}', validate=False).top_p == 1.5
    with pytest.raises(lily.LilyError):
        rq.sampling_defaults(b'{"top_p": ')


def test_chat_request_fields_parse_the_agent_surface(lily, rq):
    # tests/unit/serve.rs:133-158 (the members this layer reads; the rest is skipped)
    body = json.dumps({
        "model": "anything",
        "messages": [{"role": "system", "content": "be terse"},
                     {"role": "user", "content": [{"type": "text", "text": "hi"}]},
                     {"role": "assistant", "content": None, "tool_calls": [
                         {"id": "c1", "type": "function", "function": {"name": "f", "arguments": "{\"a\": 1}"}}]},
                     {"role": "tool", "tool_call_id": "c1", "content": "ok"}],
        "tools": [{"type": "function", "function": {"name": "f", "parameters": {"type": "object"}}}],
        "tool_choice": "auto", "temperature": 0.7, "top_p": 0.9, "top_k": 40, "seed": 5,
        "stream": True, "stream_options": {"include_usage": True}, "max_completion_tokens": 100,
        "stop": ["END"], "reasoning_effort": "low", "chat_template_kwargs": {"enable_thinking": True},
        "prompt_cache_key": "k", "user": "ignored", "parallel_tool_calls": True, "logit_bias": {},
    }).encode()
    f = rq.fields_from_json(body)
    assert f.has(rq.HAS_TOP_K) and f.top_k == 40
    assert f.has(rq.HAS_SEED) and f.seed == 5
    assert abs(f.temperature - 0.7) < 1e-6 and abs(f.top_p - 0.9) < 1e-6
    assert not f.has(rq.HAS_MIN_P) and not f.has(rq.HAS_THINKING_BUDGET)


def test_resolve_sampling_over_the_defaults(lily, rq):
    # src/serve/api.rs:798-834
    defaults = rq.sampling_defaults(b'{"temperature": 0.6, "top_k": 20, "top_p": 0.95}')
    p = rq.resolve_sampling(rq.fields_from_json(b'{}'), defaults, entropy=77)
    assert (round(p.temperature, 6), p.top_k, round(p.top_p, 6), p.seed) == (0.6, 20, 0.95, 77)
    p = rq.resolve_sampling(rq.fields_from_json(b'{"top_k": -1, "seed": 9, "min_p": 0.1}'), defaults)
    assert (p.top_k, p.seed, round(p.min_p, 6)) == (0, 9, 0.1)  # a negative top_k means off
    p = rq.resolve_sampling(rq.fields_from_json(b'{"seed": -1}'), defaults)
    assert p.seed == 2**64 - 1  # the i64 is taken as a u64
    p = rq.resolve_sampling(rq.fields_from_json(b'{"temperature": null, "top_k": 0}'), defaults)
    assert (round(p.temperature, 6), p.top_k) == (0.6, 0)  # null is "not set"
    with pytest.raises(lily.LilyError):
        rq.resolve_sampling(rq.fields_from_json(b'{"top_p": 0}'), defaults)
    with pytest.raises(lily.LilyError):
        rq.resolve_sampling(rq.fields_from_json(b'{"repetition_penalty": 0}'), defaults)
    with pytest.raises(lily.LilyError):
        rq.fields_from_json(b'{"temperature": "hot"}')
    with pytest.raises(lily.LilyError):
        rq.fields_from_json(b'{"top_k": 1.5}')
    # The resolved parameters are what the sampler validates as well.
    assert lily.lib().lily_params_validate(p) == 0


def test_thinking_budgets_parse_per_effort_or_for_all(lily, rq):
    # tests/unit/serve/api.rs:131-151
    assert rq.thinking_budgets("8000").as_tuple() == (8000, 8000, 8000)
    m = rq.thinking_budgets("low=4000, medium=8000,high=16000")
    assert m.as_tuple() == (4000, 8000, 16000)
    partial = rq.thinking_budgets("xhigh=12000")
    assert rq.budget_at(partial, "low") is None
    assert rq.budget_at(partial, None) == 12000  # the template's default effort is xhigh
    assert rq.budget_at(m, "medium") == 8000
    assert rq.thinking_budgets(" off ").as_tuple() == (None, None, None)
    for bad in ("max=1", "low=many", "low"):
        with pytest.raises(lily.LilyError):
            rq.thinking_budgets(bad)
    assert rq.template_effort("high") == "xhigh" and rq.template_effort("max") == "xhigh"
    assert rq.template_effort("low") == "low" and rq.template_effort("none") is None


def test_a_tool_turn_scales_the_default_budget(lily, rq):
    # tests/unit/serve/api.rs:153-164
    d = rq.ThinkingDefaults(budgets=rq.thinking_budgets("medium=8000"), tool_turn_factor=0.5)
    assert rq.default_budget(d, "medium", False) == 8000
    assert rq.default_budget(d, "medium", True) == 4000
    assert rq.default_budget(d, "low", True) is None
    assert rq.default_budget(rq.ThinkingDefaults(), None, False) is None  # off by default
    rq.validate_thinking_defaults(d)
    for bad in (dict(tool_turn_factor=0.0), dict(tool_turn_factor=101.0), dict(grace=(1 << 20) + 1)):
        with pytest.raises(lily.LilyError):
            rq.validate_thinking_defaults(rq.ThinkingDefaults(**bad))


def test_thinking_fields_override_the_defaults_and_kwargs_win(lily, rq):
    # tests/unit/serve/api.rs:166-216
    defaults = rq.ThinkingDefaults(budgets=rq.thinking_budgets("8000"), nudges=1,
                                   tool_call_ends_thinking=1, grace=64)
    s = rq.resolve_thinking(rq.fields_from_json(b'{}'), defaults, 8000, 5)
    assert (s.budget, s.grace, s.nudges, s.tool_call_ends_thinking, s.seed) == (8000, 64, 1, 1, 5)
    # A negative budget turns the default off, and the nudges with it.
    s = rq.resolve_thinking(rq.fields_from_json(b'{"thinking_budget": -1}'), defaults, 8000, 5)
    assert (s.budget, s.nudges) == (-1, 0)
    own = b'{"thinking_budget": 3000, "thinking_nudges": false, "tool_call_ends_thinking": false}'
    s = rq.resolve_thinking(rq.fields_from_json(own), defaults, 8000, 5)
    assert (s.budget, s.nudges, s.tool_call_ends_thinking) == (3000, 0, 0)
    # chat_template_kwargs win over the top-level fields.
    merged = rq.fields_from_json(
        b'{"thinking_budget": 3000, "thinking_nudges": false, "tool_call_ends_thinking": false,'
        b' "chat_template_kwargs": {"thinking_budget": 100, "tool_call_ends_thinking": true}}')
    assert (merged.thinking_budget, merged.tool_call_ends_thinking, merged.thinking_nudges) == (100, 1, 0)
    with pytest.raises(lily.LilyError):
        rq.fields_from_json(b'{"chat_template_kwargs": {"thinking_nudges": "yes"}}')
    # Off by default: no control at all (ThinkingSettings::any is false).
    none = rq.resolve_thinking(rq.fields_from_json(b'{}'), rq.ThinkingDefaults(), None, 5)
    assert lily.lib().lily_thinking_settings_any(none) == 0 or (none.budget < 0 and not none.nudges
                                                                 and not none.tool_call_ends_thinking)


def test_thinking_fields_come_from_a_chat_request(lily, rq):
    # tests/unit/serve/api.rs:218-232
    f = rq.fields_from_json(json.dumps({
        "messages": [{"role": "user", "content": "hi"}], "thinking_budget": 8000,
        "thinking_nudges": True, "tool_call_ends_thinking": True, "temperature": 0.6}).encode())
    assert (f.thinking_budget, f.thinking_nudges, f.tool_call_ends_thinking) == (8000, 1, 1)
    assert abs(f.temperature - 0.6) < 1e-6  # both flattened groups


def test_a_thinking_budget_of_zero_is_refused(lily, rq):
    # tests/unit/serve/api.rs:236-248
    with pytest.raises(lily.LilyError) as e:
        rq.fields_from_json(b'{"thinking_budget": 0}')
    assert "positive" in str(e.value)
    rq.fields_from_json(b'{"thinking_budget": -1}')  # negative turns a default off
    with pytest.raises(lily.LilyError) as e:
        rq.fields_from_json(b'{"chat_template_kwargs": {"thinking_budget": 0}}')
    assert "chat_template_kwargs.thinking_budget" in str(e.value)
    for bad in ("0", "low=0,medium=8000"):
        with pytest.raises(lily.LilyError):
            rq.thinking_budgets(bad)
    assert rq.thinking_budgets("low=1").as_tuple() == (1, None, None)


def test_resolved_settings_drive_the_thinking_control(lily, rq):
    """The two halves meet: a request's fields resolve into the settings the
    thinking control is built from."""
    d = rq.ThinkingDefaults(budgets=rq.thinking_budgets("low=16"), grace=4)
    f = rq.fields_from_json(b'{"reasoning_effort": "low", "thinking_nudges": true}')
    effort = rq.template_effort("low")
    s = rq.resolve_thinking(f, d, rq.default_budget(d, effort, False), seed=3)
    assert (s.budget, s.grace, s.nudges) == (16, 4, 1)
    assert lily.lib().lily_thinking_settings_any(s) == 1
