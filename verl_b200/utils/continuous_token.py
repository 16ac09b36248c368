"""Token-level continuation of a multi-turn conversation.

In a multi-turn rollout the model's own tokens must be kept exactly as they were sampled: re-rendering the whole
conversation through the chat template after every turn may tokenise an assistant turn differently from what was generated
(and what the log-probs belong to). :class:`ContinuousTokenBuilder` therefore renders only what the template ADDS for the new
non-assistant messages (tool results, user turns) and the next assistant header, by rendering them behind a short synthetic
context and cutting that context off:

    appended = render(dummy_context + new_messages, generation prompt)[len(render(dummy_context, trimmed to the stop shape)):]

"Trimmed to the stop shape" means the synthetic assistant turn ends where generation stops (at the end-of-turn token), so
whatever the template writes after that token (a newline, usually) belongs to the appended run. :func:`check_append_only`
tests a tokenizer / template for the property this relies on.

Reference: ``verl/utils/tokenizer/continuous_token.py:57-1393`` (ContinuousToken builders) and
``scripts/chat_template_checker.py`` (append-only checks over mock trajectories).
"""

from __future__ import annotations

from typing import Optional, Sequence

__all__ = ["ContinuousTokenBuilder", "check_append_only", "MOCK_TRAJECTORIES"]


def _ids(x) -> list:
    return list(x["input_ids"] if isinstance(x, dict) else x)


class ContinuousTokenBuilder:
    def __init__(self, tokenizer, tools: Optional[list] = None, dummy_context: Optional[list] = None, template_kwargs: Optional[dict] = None):
        self.tokenizer, self.tools = tokenizer, tools
        self.kw = dict(template_kwargs or {})
        self.dummy = list(dummy_context) if dummy_context is not None else [{"role": "user", "content": "."}, {"role": "assistant", "content": "."}]
        self._prefix = self._stop_shape(self._render(self.dummy, generation_prompt=False))

    def _render(self, messages: Sequence[dict], generation_prompt: bool) -> list:
        return _ids(self.tokenizer.apply_chat_template(list(messages), tools=self.tools, add_generation_prompt=generation_prompt, tokenize=True, **self.kw))

    def _stop_shape(self, ids: list) -> list:
        """Cut a rendered conversation that ends with an assistant turn right after its end-of-turn token."""
        eos = getattr(self.tokenizer, "eos_token_id", None)
        if eos is None or eos not in ids:
            return ids
        last = len(ids) - 1 - ids[::-1].index(eos)
        return ids[: last + 1]

    # ------------------------------------------------------------------ public
    def initial_prompt(self, messages: Sequence[dict]) -> list:
        """Prompt tokens of the conversation so far, ending with the assistant header."""
        return self._render(messages, generation_prompt=True)

    def merge_context_tokens(self, token_ids: list, new_messages: Sequence[dict], generation_prompt: bool = True) -> list:
        """``token_ids`` (a conversation that stopped at an assistant's end-of-turn token, or was cut by the length limit)
        extended by what the template adds for ``new_messages`` (+ the next assistant header)."""
        full = self._render(self.dummy + list(new_messages), generation_prompt)
        n = len(self._prefix)
        if full[:n] != self._prefix:
            raise ValueError("the chat template does not render the synthetic context as a prefix of the extended conversation; "
                             "pass a dummy_context that it renders append-only")
        appended = full[n:]
        eos = getattr(self.tokenizer, "eos_token_id", None)
        if token_ids and eos is not None and token_ids[-1] != eos:
            appended = [eos] + appended            # generation was cut before the end-of-turn token: close the turn first
        return list(token_ids) + appended

    def response_mask_for(self, n_generated: int, n_appended: int) -> list:
        return [1] * n_generated + [0] * n_appended


# conversations exercised by the append-only check: plain chat, tool use with one and with parallel results, a user follow-up
MOCK_TRAJECTORIES = {
    "single_turn": [{"role": "user", "content": "What is 2 + 2?"}, {"role": "assistant", "content": "4"}],
    "system_multi_turn": [{"role": "system", "content": "Be brief."}, {"role": "user", "content": "Name a prime."},
                          {"role": "assistant", "content": "7"}, {"role": "user", "content": "Another one."}, {"role": "assistant", "content": "11"}],
    "tool_call": [{"role": "user", "content": "Weather in Paris?"},
                  {"role": "assistant", "content": '<tool_call>{"name": "weather", "arguments": {"city": "Paris"}}</tool_call>'},
                  {"role": "tool", "content": "18C, cloudy"}, {"role": "assistant", "content": "It is 18C and cloudy."}],
    "parallel_tools": [{"role": "user", "content": "Compare Paris and Rome."},
                       {"role": "assistant", "content": '<tool_call>{"name": "weather", "arguments": {"city": "Paris"}}</tool_call>'},
                       {"role": "tool", "content": "18C"}, {"role": "tool", "content": "24C"},
                       {"role": "assistant", "content": "Rome is warmer."}, {"role": "user", "content": "By how much?"},
                       {"role": "assistant", "content": "6 degrees."}],
}


def check_append_only(tokenizer, trajectories: Optional[dict] = None, tools: Optional[list] = None, template_kwargs: Optional[dict] = None) -> dict:
    """Two checks per trajectory (the reference checker's layers):

    1. ``raw_prefix``: rendering a prefix of the conversation gives a token prefix of rendering more of it (a diagnostic —
       the builder does not need it globally);
    2. ``builder``: at every boundary where non-assistant messages follow an assistant turn, the prefix rendered up to that
       turn (stop shape) merged with the following run by :class:`ContinuousTokenBuilder` equals a single render of the same
       messages with a generation prompt.

    → ``{name: {"raw_prefix": bool, "builder": bool, "boundaries": int, "detail": str}}``"""
    kw = dict(template_kwargs or {})
    b = ContinuousTokenBuilder(tokenizer, tools=tools, template_kwargs=kw)
    report = {}
    for name, msgs in (trajectories or MOCK_TRAJECTORIES).items():
        raw_ok, builder_ok, nb, detail = True, True, 0, ""
        prev = None
        for k in range(1, len(msgs) + 1):
            cur = _ids(tokenizer.apply_chat_template(msgs[:k], tools=tools, add_generation_prompt=False, tokenize=True, **kw))
            if prev is not None and cur[: len(prev)] != prev:
                raw_ok = False
                detail = detail or f"render of the first {k - 1} messages is not a prefix of the first {k}"
            prev = cur
        i = 0
        while i < len(msgs):
            if msgs[i]["role"] == "assistant" and i + 1 < len(msgs) and msgs[i + 1]["role"] != "assistant":
                j = i + 1
                while j < len(msgs) and msgs[j]["role"] != "assistant":
                    j += 1
                nb += 1
                prefix = b._stop_shape(_ids(tokenizer.apply_chat_template(msgs[: i + 1], tools=tools, add_generation_prompt=False, tokenize=True, **kw)))
                try:
                    merged = b.merge_context_tokens(prefix, msgs[i + 1:j])
                except ValueError as e:
                    builder_ok, detail = False, detail or str(e)
                    break
                want = _ids(tokenizer.apply_chat_template(msgs[:j], tools=tools, add_generation_prompt=True, tokenize=True, **kw))
                if merged != want:
                    builder_ok = False
                    detail = detail or f"merge after message {i} differs from the single-pass render at token {next((t for t, (x, y) in enumerate(zip(merged, want)) if x != y), min(len(merged), len(want)))}"
                i = j
            else:
                i += 1
        report[name] = {"raw_prefix": raw_ok, "builder": builder_ok, "boundaries": nb, "detail": detail}
    return report
