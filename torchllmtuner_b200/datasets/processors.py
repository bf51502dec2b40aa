"""Sample processors: raw rows -> `TextSequence` (tokens, shifted labels, positions, document ids)
(reference: llmtuner/datasets/text/processors.py:43-295, renderer.py:37-132, recipes.py:25-164)."""
from __future__ import annotations

from .contracts import IGNORE_INDEX, TextSequence


def _shifted(tokens: list[int], loss_mask: list[bool]) -> list[int]:
    """labels[t] = tokens[t+1] where the predicted token carries loss, else IGNORE_INDEX."""
    out = [IGNORE_INDEX] * len(tokens)
    for t in range(len(tokens) - 1):
        if loss_mask[t + 1]:
            out[t] = tokens[t + 1]
    return out


class TextProcessor:
    """Plain language-model rows: every token after the first carries loss."""

    def __init__(self, tokenizer, text_field: str = "text"):
        self.tok, self.field = tokenizer, text_field

    def __call__(self, row: dict) -> TextSequence:
        ids = self.tok.encode(str(row[self.field]), add_bos=self.tok.bos_id is not None, add_eos=True)
        return TextSequence(ids, _shifted(ids, [True] * len(ids)), list(range(len(ids))), [0] * len(ids))


class ChatProcessor:
    """Supervised fine-tuning rows. Single turn: prompt/response fields, loss on the response only. Multi turn: a list
    of {role, content} messages rendered with the chat template, loss on assistant turns only (found by rendering the
    conversation prefix by prefix, which is template-agnostic)."""

    def __init__(self, tokenizer, prompt_field="prompt", response_field="response", messages_field="messages", multiturn=False,
                 template_kwargs=None):
        self.tok, self.pf, self.rf, self.mf, self.multiturn = tokenizer, prompt_field, response_field, messages_field, multiturn
        self.kw = template_kwargs or {}

    def __call__(self, row: dict) -> TextSequence:
        if self.multiturn or self.mf in row:
            msgs = row[self.mf]
        else:
            msgs = [{"role": "user", "content": str(row[self.pf])}, {"role": "assistant", "content": str(row[self.rf])}]
        ids: list[int] = []
        mask: list[bool] = []
        for i, m in enumerate(msgs):
            upto = self.tok.encode(self.tok.apply_chat_template(msgs[:i + 1], **self.kw))
            if upto[:len(ids)] != ids:          # template is not prefix-stable: fall back to whole-conversation loss
                ids, mask = upto, [True] * len(upto)
                continue
            new = upto[len(ids):]
            mask += [m["role"] == "assistant"] * len(new)
            ids = upto
        return TextSequence(ids, _shifted(ids, mask), list(range(len(ids))), [0] * len(ids))
