"""Host-side pieces of the serving shim that need no GPU: chat-template tokenisation (src/server.py:72-85) and the
conversion of text records into token-id records."""
import os
import sys
import types

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "..", "open-jev-fast_b200"))

from ojb200 import server as SV


class _Backend:
    def __init__(self, owner):
        self.owner = owner
        self.calls = 0

    def encode_batch(self, texts, add_special_tokens=True):
        self.calls += 1
        return [types.SimpleNamespace(ids=self.owner.encode(t)) for t in texts]


class _Tok:
    """Character-level stand-in for a Hugging Face tokenizer with a chat template."""

    def __init__(self, head="<|user|>", tail="<|assistant|>", echo_twice=False):
        self.head, self.tail, self.echo_twice = head, tail, echo_twice
        self.backend_tokenizer = _Backend(self)
        self.renders = 0

    def encode(self, text):
        return [ord(c) for c in text]

    def apply_chat_template(self, messages, tokenize=False, add_generation_prompt=True, enable_thinking=False):
        assert not tokenize and add_generation_prompt and not enable_thinking and len(messages) == 1
        self.renders += 1
        body = messages[0]["content"]
        return self.head + body + (body if self.echo_twice else "") + self.tail

    def __call__(self, text):
        return {"input_ids": self.encode(text)}


def test_prompt_ids_batches_through_the_cached_template():
    tok = _Tok()
    prompts = ["alpha", "", "b c"]
    ids = SV.prompt_ids(tok, prompts)
    assert ids == [tok.encode(tok.head + p + tok.tail) for p in prompts]
    assert tok.renders == 1 and tok.backend_tokenizer.calls == 1
    SV.prompt_ids(tok, ["again"])
    assert tok.renders == 1 and tok.backend_tokenizer.calls == 2      # the template is rendered once per tokenizer


def test_prompt_ids_falls_back_when_the_marker_is_not_unique():
    tok = _Tok(echo_twice=True)
    prompts = ["x", "yz"]
    ids = SV.prompt_ids(tok, prompts)
    assert ids == [tok.encode(tok.head + p + p + tok.tail) for p in prompts]
    assert tok.backend_tokenizer.calls == 0 and tok.renders == 1 + len(prompts)


def test_token_records_keep_order_kind_and_counts():
    tok = _Tok()
    records = [{"kind": "noul", "q": "is it", "opts": ["yes"]}, {"kind": "choice", "q": "which", "opts": ["a", "b", "c"]}]
    out = SV.token_records(records, tok, lambda r: [r["q"] + " " + o for o in r["opts"]])
    assert [r["kind"] for r in out] == ["noul", "choice"]
    assert [len(r["candidates"]) for r in out] == [1, 3]
    assert out[1]["candidates"][2] == tok.encode(tok.head + "which c" + tok.tail)
    assert tok.backend_tokenizer.calls == 1                            # one batched encode for the whole request
