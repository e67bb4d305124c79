"""A stand-in tokenizer for the command line.

The engine's interface is token ids.  The reference ships its own byte-level BPE
with a chat template (serving/tokenizer.py, serving/bpe.py); that is text handling
before a request's tokens exist and is not part of this engine.  For ``--chat TEXT``
the command line maps UTF-8 bytes to ids (in the manner of the reference's
``TinyCharTokenizer``, serving/dev_model.py:433-454), which is meaningful only for
random or byte-vocabulary models; with real checkpoints pass ``--prompt-ids``.
"""

from __future__ import annotations


class ByteTokenizer:
    def __init__(self, vocab_size: int):
        self.vocab_size = int(vocab_size)

    def encode(self, text: str) -> list[int]:
        return [b % self.vocab_size for b in text.encode("utf-8")] or [0]

    def decode(self, ids) -> str:
        return bytes(int(i) % 256 for i in ids).decode("utf-8", errors="replace")
