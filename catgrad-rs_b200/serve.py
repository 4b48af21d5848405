"""The serving interfaces of catgrad-llm/src/serve.rs over the fused decoder.

`LM` mirrors `trait LM<T>: Iterator<Item = T>` (serve.rs:12-20): a language model has a settable
context and yields new tokens one at a time; `complete(context)` sets the context and returns the
iterator.  `DecoderLM` implements it the way the reference's `ModelRunner` does
(catgrad-llm/src/run.rs:262-305) -- every `next` runs the tokens not yet in the KV cache and
returns the greedy next token, `None` (StopIteration) at an end-of-sequence token -- with two
differences: the cache lives on the device inside the decoder instead of being passed in and out
of the graph, and `set_context` keeps the longest common prefix of the old and the new context
(the reference keeps its cache only when the new context extends the whole old one, and says so
in a PERFORMANCE note at run.rs:296).  `Tokenizer` / `ChatTokenizer` / `Loader` are the
abstract interfaces only: tokenizers are outside this library.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from .decoder import Decoder


@dataclass
class Message:
    """serve.rs:4-9"""
    role: str
    content: str


class LM:
    """serve.rs:11-20"""

    def set_context(self, context):
        raise NotImplementedError

    def __iter__(self):
        return self

    def __next__(self):
        raise NotImplementedError

    def complete(self, context):
        self.set_context(context)
        return self


class Tokenizer:
    """serve.rs:29-33"""

    def encode(self, content: str):
        raise NotImplementedError

    def decode(self, tokens) -> str:
        raise NotImplementedError


class ChatTokenizer:
    """serve.rs:35-38"""

    def encode_messages(self, messages):
        raise NotImplementedError


class Loader:
    """serve.rs:22-27"""

    def load_runner(self) -> LM:
        raise NotImplementedError

    def load_tokenizer(self) -> Tokenizer:
        raise NotImplementedError


def longest_common_prefix(x, y) -> int:
    """run.rs:270-280"""
    n = 0
    for a, b in zip(x, y):
        if a != b:
            break
        n += 1
    return n


class DecoderLM(LM):
    """One sequence (batch 1) on a finalized `Decoder`."""

    def __init__(self, decoder: Decoder, eos_token_ids=()):
        self.dec = decoder
        self.B = decoder.B
        self.eos = set(int(t) for t in eos_token_ids)
        self.context: list[int] = []   # everything the model has been asked to condition on
        self.cached: list[int] = []    # the tokens whose keys and values are in the cache
        self.pending: list[int] = []   # tokens to run at the next step

    def set_context(self, context):
        context = [int(t) for t in context]
        n = longest_common_prefix(self.cached, context)
        if n == len(context) and n > 0:
            n -= 1                      # at least one token must be run to get a next token
        if n < len(self.cached):
            self.dec.truncate(n)        # forget only what differs
            self.cached = self.cached[:n]
        self.context = context
        self.pending = context[n:]

    def __next__(self) -> int:
        if not self.pending:
            raise StopIteration
        toks = self.B.from_numpy(np.asarray(self.pending, dtype=np.uint32).reshape(1, -1))
        self.dec.append(toks)
        self.cached += self.pending
        token = int(self.dec.tokens()[0, -1])
        if token in self.eos:           # EOS tokens are not emitted (run.rs:252-255)
            self.pending = []
            raise StopIteration
        self.context.append(token)
        self.pending = [token]
        return token
