"""Incremental detokenisation reads the end of the prompt as context: a SentencePiece-style tokenizer writes the
space before a word only when another token precedes it, so the first generated word needs the prompt behind it."""
from types import SimpleNamespace

import numpy as np

from lightllm_b200.server.detokenization.decode import DecodeReq, decode_token, prompt_context_len


def _metaspace_tokenizer():
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast

    words = ["<unk>", "<s>", "</s>", "▁Hello", "▁world", "▁again", "!", "▁", "▁Gr", "ü", "ße"]
    tok = Tokenizer(models.WordLevel({w: i for i, w in enumerate(words)}, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Metaspace()
    tok.decoder = decoders.Metaspace()
    return PreTrainedTokenizerFast(tokenizer_object=tok, unk_token="<unk>", bos_token="<s>", eos_token="</s>")


def _req(prompt, **sp):
    arr = np.zeros(64, dtype=np.int64)
    arr[:len(prompt)] = prompt
    sample = SimpleNamespace(stop_sequences=SimpleNamespace(to_strings=lambda: []), skip_special_tokens=True,
                             add_spaces_between_special_tokens=False, print_eos_token=False, **sp)
    return SimpleNamespace(request_id=1, group_req_id=1, input_len=len(prompt), sample_params=sample,
                           shm_prompt_ids=SimpleNamespace(arr=arr))


def test_first_generated_word_keeps_its_space(monkeypatch):
    tk = _metaspace_tokenizer()
    assert tk.decode([4]) == "world"                      # alone, the decoder strips the leading space
    monkeypatch.delenv("LLB_DECODE_PREFIX_LENGTH", raising=False)
    monkeypatch.delenv("LIGHTLLM_DECODE_PREFIX_LENGTH", raising=False)
    assert prompt_context_len() == 5
    d = DecodeReq(_req([1, 3]))                           # "<s> Hello"
    out = [decode_token(tk, d, t, eos_ids=(2,)) for t in (4, 5, 6, 2)]
    assert out == [" world", " again", "!", ""] and d.output_ids == [4, 5, 6, 2]
    # without context (the knob at 0) the first space is lost
    monkeypatch.setenv("LIGHTLLM_DECODE_PREFIX_LENGTH", "0")
    d0 = DecodeReq(_req([1, 3]))
    assert [decode_token(tk, d0, t, eos_ids=(2,)) for t in (4, 5)] == ["world", " again"]
    monkeypatch.setenv("LLB_DECODE_PREFIX_LENGTH", "3")
    assert prompt_context_len() == 3


def test_virtual_picture_ids_at_the_end_of_a_prompt_are_not_decoded():
    tk = _metaspace_tokenizer()
    d = DecodeReq(_req([1, 3, 100_000_000, 100_000_001, 6]))      # ... picture ... "!"
    assert d.prompt_tail == [1, 3, 100_000_000, 100_000_001, 6]
    assert decode_token(tk, d, 4, eos_ids=(2,)) == " world"       # context is "!" only
    assert d.context_ids == [6, 4]
    d2 = DecodeReq(_req([3, 100_000_000]))                         # the prompt ends with the picture: no context
    assert decode_token(tk, d2, 4, eos_ids=(2,)) == "world" and d2.context_ids == [4]


def test_multibyte_pieces_wait_for_completion():
    class Bytes:
        def __len__(self):
            return 256

        def decode(self, ids, **kw):
            return bytes(ids).decode("utf-8", errors="replace")

    d = DecodeReq(_req(list(b"ab")))
    got = [decode_token(Bytes(), d, t, eos_ids=()) for t in "ü!".encode()]
    assert got == ["", "ü", "!"]
