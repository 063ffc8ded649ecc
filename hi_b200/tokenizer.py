"""Text in and out, as a convenience of the command line: the model folder's ``tokenizer.json``
through the ``tokenizers`` package, as the reference loads it (crates/hi-mlx/src/generate.rs:9-27:
encode without special tokens added, decode with special tokens skipped). Token ids are the
engine's interface; nothing in it depends on this module, and it is optional: without the
package or the file, text is simply not available."""
from __future__ import annotations

import os
from typing import List, Optional, Sequence


class TokenizerRuntime:
    def __init__(self, inner):
        self._inner = inner

    @staticmethod
    def load(model_dir: str) -> Optional["TokenizerRuntime"]:
        """The tokenizer of a model folder, or None if the folder has no ``tokenizer.json`` or the
        ``tokenizers`` package is not installed."""
        path = os.path.join(model_dir, "tokenizer.json")
        if not os.path.isfile(path):
            return None
        try:
            import tokenizers
        except ImportError:
            return None
        return TokenizerRuntime(tokenizers.Tokenizer.from_file(path))

    def encode(self, text: str) -> List[int]:
        return list(self._inner.encode(text, add_special_tokens=False).ids)

    def decode(self, tokens: Sequence[int]) -> str:
        return self._inner.decode(list(tokens), skip_special_tokens=True)

    def token(self, token_id: int) -> Optional[str]:
        return self._inner.id_to_token(int(token_id))
