"""The reference's tokenizer file format, its BPE merge rule and its chat protocol, on CPU.

The real Qwen2 vocabulary is not available offline, so the vocabulary here is a small byte-level BPE trained on the
spot with the `tokenizers` library (the Hugging Face implementation the reference's converter reads its input from,
tools/qwen2_convert.py:176-217); the merge rule is checked against that library run WITHOUT pre-tokenisation, and
against the reference's own loop restated literally (scan, merge the leftmost pair of lowest rank, shift, repeat:
lean/algorithms/Qwen2Common.lean:1132-1258)."""
import json
import random

import pytest

from base_b200.chat import ASSISTANT, IM_END, IM_START, NEWLINE, USER, ChatSession
from base_b200.tokenizer import Tokenizer, gpt2_byte_decoder

CORPUS = ["the quick brown fox jumps over the lazy dog", "hello there, how are you today?", "hello! how can i assist you today?",
          "a aa aaa aaaa banana bandana", "tokens, tokenizers and tokenisation", "  spaces   and\ttabs\nnewlines\n",
          "naïve café über straße", "日本語のテキスト", "1234567890 + 0987654321 = ?"] * 3


def train_hf(vocab_size=400):
    tokenizers = pytest.importorskip("tokenizers")
    from tokenizers import Tokenizer as HfTokenizer, decoders, models, pre_tokenizers, trainers
    hf = HfTokenizer(models.BPE())
    hf.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)      # no split: whole text
    hf.decoder = decoders.ByteLevel()
    trainer = trainers.BpeTrainer(vocab_size=vocab_size, initial_alphabet=pre_tokenizers.ByteLevel.alphabet(), show_progress=False)
    hf.train_from_iterator(CORPUS, trainer)
    return hf


@pytest.fixture(scope="module")
def pair():
    hf = train_hf()
    tok = Tokenizer.from_hf_json(json.loads(hf.to_str()))
    return hf, tok


def samples():
    rng = random.Random(5)
    out = list(CORPUS[:9]) + ["", "a", "aa", "aaaaaaa", "the the the", "thethethe"]
    alphabet = "abcdehlnorstuy ,.!?\n"
    out += ["".join(rng.choice(alphabet) for _ in range(rng.randrange(1, 60))) for _ in range(200)]
    out += [bytes(rng.randrange(256) for _ in range(rng.randrange(1, 40))) for _ in range(50)]      # arbitrary bytes
    return out


def test_byte_alphabet_is_a_bijection():
    dec = gpt2_byte_decoder()
    assert len(dec) == 256 and sorted(dec.values()) == list(range(256))
    assert dec["A"] == ord("A") and dec["Ġ"] == ord(" ") and dec["Ċ"] == ord("\n")


def test_heap_encoder_equals_the_reference_loop_and_round_trips(pair):
    _, tok = pair
    assert tok.vocab_size >= 256 and len(tok.merges) > 50
    for s in samples():
        ids = tok.encode(s)
        assert ids == tok.encode_by_rescan(s), s
        raw = s.encode("utf-8") if isinstance(s, str) else s
        assert tok.decode_bytes(ids) == raw


def test_encoder_equals_hugging_face_bpe_without_pretokenisation(pair):
    hf, tok = pair
    for s in samples():
        if isinstance(s, bytes):
            continue
        assert tok.encode(s) == hf.encode(s).ids, s


def test_file_format_round_trip_and_layout(pair, tmp_path):
    import struct
    _, tok = pair
    blob = tok.to_bytes()
    n_merges, vocab, pool, zero = struct.unpack_from("<4I", blob, 0)
    assert (n_merges, vocab, zero) == (len(tok.merges), tok.vocab_size, 0)
    assert len(blob) == 1040 + 12 * n_merges + 8 * vocab + pool
    assert struct.unpack_from("<3I", blob, 1040) == tok.merges[0]              # the merge table starts at byte 1040
    assert struct.unpack_from("<I", blob, 16 + 4 * ord("a"))[0] == tok.byte_init[ord("a")]
    p = tmp_path / "tok.bin"
    tok.save(str(p))
    back = Tokenizer.load(str(p))
    assert back.merges == tok.merges and back.byte_init == tok.byte_init and back.token_bytes == tok.token_bytes
    with pytest.raises(ValueError):
        Tokenizer.from_bytes(blob[:-1])
    with pytest.raises(ValueError):
        Tokenizer(tok.byte_init, list(tok.merges) + [tok.merges[0]], tok.token_bytes)       # a pair listed twice


class Scripted:
    """A decoder that records what it is fed and answers from a script once the prompt's last token has arrived."""

    def __init__(self, answers):
        self.fed, self.answers, self.turn, self.k = [], answers, 0, 0

    def step(self, token, pos):
        assert pos == len(self.fed)                      # positions are consecutive over the whole conversation
        self.fed.append(token)
        if token == NEWLINE and len(self.fed) >= 11 and self.fed[-11:-1] == [IM_START, *ASSISTANT]:
            self.k = 0                                   # generation of this turn starts after `assistant\n`
        script = self.answers[min(self.turn, len(self.answers) - 1)]
        out = script[self.k] if self.k < len(script) else IM_END
        self.k += 1
        return out


def test_chat_turn_follows_the_reference_protocol(pair):
    _, tok = pair
    hello = tok.encode("hello!")
    dec = Scripted([hello + [IM_END], tok.encode("ok") + [151643]])
    system = [IM_START, 5, 6, IM_END, NEWLINE]
    chat = ChatSession(dec.step, tok, max_seq=512, system_tokens=system)
    assert dec.fed == system and chat.pos == len(system)
    reply = chat.turn(b"hi there")
    body = tok.encode(b"hi there")
    want = system + [IM_START, *USER, NEWLINE] + body + [IM_END, NEWLINE, IM_START, *ASSISTANT, NEWLINE] + hello + [IM_END, NEWLINE]
    assert reply == b"hello!\n"
    assert dec.fed == want                               # the stop token itself is not fed as a generated token; the closing pair is
    assert len([IM_START, *USER, NEWLINE]) == 6 and len([IM_END, NEWLINE, IM_START, *ASSISTANT, NEWLINE]) == 13
    dec.turn = 1
    assert chat.turn(b"again") == b"ok\n" and chat.pos == len(dec.fed)


def test_chat_stops_at_the_budget_and_refuses_what_cannot_fit(pair):
    _, tok = pair
    a = tok.encode("a")[0]
    dec = Scripted([[a] * 1000])
    chat = ChatSession(dec.step, tok, max_seq=256, system_tokens=[IM_START, NEWLINE], max_decode=16)
    assert chat.turn(b"x") == b"a" * 16 + b"\n"
    assert chat.max_recv == 256 - 2 - 19 - 16
    with pytest.raises(ValueError):
        chat.turn(b"y" * (chat.max_recv + 1))
    with pytest.raises(ValueError):                      # the context fills up over the turns
        for _ in range(20):
            chat.turn(b"z" * 40)
