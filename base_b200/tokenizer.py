"""Byte-level BPE tokenizer in the reference's own file format and with its merge rule.

File format (tools/qwen2_convert.py:176-232 writes it, lean/algorithms/Qwen2Common.lean:1059-1070 reads it), little endian:

    [0]     n_merges:u32  vocab_size:u32  byte_pool_size:u32  0:u32
    [16]    byte_init[256]:u32                    token id of every single byte
    [1040]  merges[n_merges] x (tok_a:u32, tok_b:u32, result:u32)      rank = index
    ...     decode_offsets[vocab_size]:u32, decode_lens[vocab_size]:u32, byte_pool

Encoding (Qwen2Common.lean:1112-1258): one token per input byte, then, until no adjacent pair is in the merge table,
the pair of lowest rank is merged, the leftmost one when several positions share that rank.  There is NO
pre-tokenisation (no regular expression split): merges may cross what other tokenisers treat as word boundaries.
Decoding concatenates the tokens' byte strings.  `encode` below gives exactly that result with a heap instead of a
rescan per merge.
"""
from __future__ import annotations

import heapq
import struct
from typing import Dict, Iterable, List, Sequence, Tuple


def gpt2_byte_decoder() -> Dict[str, int]:
    """{unicode character: byte value} of the GPT-2 byte-level alphabet (the printable bytes stand for themselves,
    the others are mapped to U+0100 onwards in byte order)."""
    keep = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAD)) + list(range(0xAE, 0x100))
    chars = keep[:]
    extra = 0
    for b in range(256):
        if b not in keep:
            keep.append(b)
            chars.append(256 + extra)
            extra += 1
    return {chr(c): b for b, c in zip(keep, chars)}


class Tokenizer:
    def __init__(self, byte_init: Sequence[int], merges: Sequence[Tuple[int, int, int]], token_bytes: Sequence[bytes]):
        if len(byte_init) != 256:
            raise ValueError("byte_init must have 256 entries")
        self.byte_init = [int(t) for t in byte_init]
        self.merges = [(int(a), int(b), int(r)) for a, b, r in merges]
        self.token_bytes = [bytes(b) for b in token_bytes]
        self.vocab_size = len(self.token_bytes)
        # first rank wins if a pair is listed twice, as a hash table that is filled in rank order and never overwritten
        # would; the reference's table is insert-or-update, so a file with duplicate pairs is refused instead
        self.rank: Dict[Tuple[int, int], Tuple[int, int]] = {}
        for i, (a, b, r) in enumerate(self.merges):
            if (a, b) in self.rank:
                raise ValueError(f"merge pair ({a}, {b}) listed twice")
            if max(a, b, r) >= self.vocab_size:
                raise ValueError("merge refers to a token outside the vocabulary")
            self.rank[(a, b)] = (i, r)

    # ---- file format ------------------------------------------------------------------------------------
    @classmethod
    def from_bytes(cls, blob: bytes) -> "Tokenizer":
        if len(blob) < 1040:
            raise ValueError("tokenizer file too short")
        n_merges, vocab, pool, _ = struct.unpack_from("<4I", blob, 0)
        need = 1040 + 12 * n_merges + 8 * vocab + pool
        if len(blob) < need:
            raise ValueError(f"tokenizer file too short: {len(blob)} bytes, header asks for {need}")
        byte_init = struct.unpack_from("<256I", blob, 16)
        merges = [struct.unpack_from("<3I", blob, 1040 + 12 * i) for i in range(n_merges)]
        off0 = 1040 + 12 * n_merges
        offs = struct.unpack_from(f"<{vocab}I", blob, off0)
        lens = struct.unpack_from(f"<{vocab}I", blob, off0 + 4 * vocab)
        base = off0 + 8 * vocab
        toks = []
        for o, n in zip(offs, lens):
            if o + n > pool:
                raise ValueError("token bytes outside the byte pool")
            toks.append(blob[base + o:base + o + n])
        return cls(byte_init, merges, toks)

    @classmethod
    def load(cls, path: str) -> "Tokenizer":
        with open(path, "rb") as f:
            return cls.from_bytes(f.read())

    def to_bytes(self) -> bytes:
        pool = bytearray()
        offs, lens = [], []
        for b in self.token_bytes:
            offs.append(len(pool))
            lens.append(len(b))
            pool += b
        out = bytearray(struct.pack("<4I", len(self.merges), self.vocab_size, len(pool), 0))
        out += struct.pack("<256I", *self.byte_init)
        for m in self.merges:
            out += struct.pack("<3I", *m)
        out += struct.pack(f"<{self.vocab_size}I", *offs)
        out += struct.pack(f"<{self.vocab_size}I", *lens)
        out += pool
        return bytes(out)

    def save(self, path: str) -> None:
        with open(path, "wb") as f:
            f.write(self.to_bytes())

    @classmethod
    def from_hf_json(cls, tok: dict) -> "Tokenizer":
        """From a parsed Hugging Face `tokenizer.json` (byte-level BPE), the conversion of tools/qwen2_convert.py:176-217:
        vocabulary strings are in the GPT-2 byte alphabet; added tokens keep their ids and decode to their UTF-8 text."""
        model = tok["model"]
        vocab: Dict[str, int] = dict(model["vocab"])
        for added in tok.get("added_tokens", []):
            vocab.setdefault(added["content"], added["id"])
        dec = gpt2_byte_decoder()
        size = max(vocab.values()) + 1
        token_bytes = [b""] * size
        for s, i in vocab.items():
            raw = bytearray()
            for ch in s:
                if ch in dec:
                    raw.append(dec[ch])
                else:
                    raw += ch.encode("utf-8", errors="replace")
            token_bytes[i] = bytes(raw)
        byte_init = [0] * 256
        for ch, b in dec.items():
            if ch in vocab:
                byte_init[b] = vocab[ch]
        merges = []
        for m in model.get("merges", []):
            a, b = m.split(" ", 1) if isinstance(m, str) else m
            if a in vocab and b in vocab and a + b in vocab:
                merges.append((vocab[a], vocab[b], vocab[a + b]))
        return cls(byte_init, merges, token_bytes)

    # ---- encode / decode ----------------------------------------------------------------------------------
    def encode(self, text) -> List[int]:
        data = text.encode("utf-8") if isinstance(text, str) else bytes(text)
        toks = [self.byte_init[b] for b in data]
        n = len(toks)
        if n < 2:
            return toks
        # doubly linked list over the positions; heap of (rank, position of the left token, left token, right token)
        prev = list(range(-1, n - 1))
        nxt = list(range(1, n + 1))
        nxt[-1] = -1
        alive = [True] * n
        heap: List[Tuple[int, int, int, int]] = []

        def push(i: int) -> None:
            j = nxt[i]
            if j >= 0:
                hit = self.rank.get((toks[i], toks[j]))
                if hit is not None:
                    heapq.heappush(heap, (hit[0], i, toks[i], toks[j]))

        for i in range(n - 1):
            push(i)
        while heap:
            rank, i, a, b = heapq.heappop(heap)
            j = nxt[i] if alive[i] else -1
            if j < 0 or toks[i] != a or toks[j] != b:
                continue                               # a stale entry: one of the two tokens was merged away
            toks[i] = self.rank[(a, b)][1]
            alive[j] = False
            nxt[i] = nxt[j]
            if nxt[j] >= 0:
                prev[nxt[j]] = i
            if prev[i] >= 0:
                push(prev[i])
            push(i)
        return [toks[i] for i in range(n) if alive[i]]

    def encode_by_rescan(self, text) -> List[int]:
        """The reference's loop as written (scan every adjacent pair, merge the leftmost pair of lowest rank, shift,
        repeat): quadratic, for tests."""
        data = text.encode("utf-8") if isinstance(text, str) else bytes(text)
        toks = [self.byte_init[b] for b in data]
        while len(toks) > 1:
            best_rank, best_pos = None, -1
            for i in range(len(toks) - 1):
                hit = self.rank.get((toks[i], toks[i + 1]))
                if hit is not None and (best_rank is None or hit[0] < best_rank):
                    best_rank, best_pos = hit[0], i
            if best_pos < 0:
                break
            toks[best_pos:best_pos + 2] = [self.rank[(toks[best_pos], toks[best_pos + 1])][1]]
        return toks

    def decode_bytes(self, ids: Iterable[int]) -> bytes:
        out = bytearray()
        for t in ids:
            if not 0 <= t < self.vocab_size:
                raise ValueError(f"token id {t} outside the vocabulary")
            out += self.token_bytes[t]
        return bytes(out)

    def decode(self, ids: Iterable[int]) -> str:
        return self.decode_bytes(ids).decode("utf-8", errors="replace")
