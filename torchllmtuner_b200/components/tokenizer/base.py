from __future__ import annotations


class BaseTokenizer:
    """Contract: `encode(text, add_bos, add_eos) -> list[int]`, `decode(ids) -> str`, ids of the special tokens."""

    bos_id: int | None = None
    eos_id: int | None = None
    pad_id: int | None = None

    def encode(self, text: str, add_bos: bool = False, add_eos: bool = False) -> list[int]:
        raise NotImplementedError

    def decode(self, ids) -> str:
        raise NotImplementedError

    @property
    def vocab_size(self) -> int:
        raise NotImplementedError

    def apply_chat_template(self, messages: list[dict], add_generation_prompt: bool = False, **kw) -> str:
        """Default ChatML rendering; back ends with a stored template override this."""
        out = []
        for m in messages:
            out.append(f"<|im_start|>{m['role']}\n{m['content']}<|im_end|>\n")
        if add_generation_prompt:
            out.append("<|im_start|>assistant\n")
        return "".join(out)

    def identity(self) -> str:
        return f"{type(self).__name__}:{self.vocab_size}"
