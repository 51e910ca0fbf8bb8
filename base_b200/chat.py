"""The reference's chat loop (lean/algorithms/Qwen2Common.lean:187-245, 1300-1505) over any greedy decoder.

Protocol, as the reference runs it:
  * once: the pre-tokenised system prompt is fed through the model, position by position (its outputs are dropped);
  * per user line: tokens = `<|im_start|>` u s e r `\\n` + BPE(line bytes) + `<|im_end|>` `\\n` `<|im_start|>`
    a s s i s t a n t `\\n` (the role names are spelled with single-character tokens; 6 + 13 wrapper tokens); they are
    fed one per step, the prediction after the last one is the first generated token; generation stops at
    `<|endoftext|>`, at `<|im_end|>` or after MAX_DECODE tokens (the stop token is not part of the answer);
  * the answer is the decoded bytes plus a newline; then `<|im_end|>` `\\n` are fed so that the cache holds a closed
    assistant turn, and the next line continues from there.
A line that would not fit the context (system prompt + line bytes + wrapper + MAX_DECODE <= max_seq, one token per
byte being the worst case) is refused, as the reference's derived input limit does.

`python -m base_b200.chat --tokenizer FILE` runs the loop on stdin/stdout over the `native:qwen2` stage program with
the Qwen2-0.5B shapes; `--weights FILE` loads a flat f32 weight file in the reference's layout (without it the weights
are generated from a seed and the answers are noise).  The protocol is tested against a scripted decoder.
"""
from __future__ import annotations

import argparse
import sys
from typing import Callable, List, Sequence

from .tokenizer import Tokenizer

IM_START, IM_END, END_OF_TEXT, NEWLINE = 151644, 151645, 151643, 198
USER = (84, 82, 68, 81)                                  # u s e r
ASSISTANT = (64, 82, 82, 72, 82, 83, 64, 77, 83)         # a s s i s t a n t
SYSTEM_TOKENS = (151644, 8948, 198,
                 2610, 525, 264, 11657, 7517, 1663, 17847, 13, 17841, 5961, 323, 17712, 13, 14152, 279, 1196, 594,
                 16232, 1959, 421, 807, 40786, 498, 64614, 11, 40786, 1182, 64614, 13,
                 151645, 198)
MAX_DECODE = 128
PREFIX_LEN, WRAP_LEN = 6, 19


class ChatSession:
    """`step(token, position) -> next token` is the decoder (one greedy decode step; the KV cache lives behind it)."""

    def __init__(self, step: Callable[[int, int], int], tokenizer: Tokenizer, max_seq: int = 2048,
                 system_tokens: Sequence[int] = SYSTEM_TOKENS, max_decode: int = MAX_DECODE,
                 im_start: int = IM_START, im_end: int = IM_END, end_of_text: int = END_OF_TEXT, newline: int = NEWLINE,
                 user: Sequence[int] = USER, assistant: Sequence[int] = ASSISTANT):
        self.step, self.tok, self.max_seq, self.max_decode = step, tokenizer, max_seq, max_decode
        self.im_start, self.im_end, self.eot, self.nl = im_start, im_end, end_of_text, newline
        self.prefix = [im_start, *user, newline]
        self.suffix = [im_end, newline, im_start, *assistant, newline]
        self.system = list(system_tokens)
        self.max_recv = max_seq - len(self.system) - len(self.prefix) - len(self.suffix) - max_decode
        self.pos = 0
        for t in self.system:                                 # the preamble goes into the cache once
            self.step(t, self.pos)
            self.pos += 1

    def wrap(self, line: bytes) -> List[int]:
        return self.prefix + self.tok.encode(line) + self.suffix

    def turn(self, line: bytes) -> bytes:
        if len(line) > self.max_recv:
            raise ValueError(f"line of {len(line)} bytes; at most {self.max_recv} fit the context")
        prompt = self.wrap(line)
        if self.pos + len(prompt) + self.max_decode + 2 > self.max_seq:
            raise ValueError("the conversation no longer fits the context")
        nxt = 0
        for t in prompt:
            nxt = self.step(t, self.pos)
            self.pos += 1
        out: List[int] = []
        while nxt not in (self.eot, self.im_end) and len(out) < self.max_decode:
            out.append(nxt)
            nxt = self.step(nxt, self.pos)
            self.pos += 1
        for t in (self.im_end, self.nl):                      # close the assistant turn in the cache
            self.step(t, self.pos)
            self.pos += 1
        return self.tok.decode_bytes(out) + b"\n"


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--tokenizer", required=True, help="tokenizer file in the reference's format (base_b200.tokenizer)")
    ap.add_argument("--weights", help="flat f32 weight file in the reference's layout (base_b200.convert.write_qwen2_flat); "
                                      "without it the Qwen2-0.5B-shaped weights are generated from --seed and the answers are noise")
    ap.add_argument("--seed", type=int, default=3, help="seed of the generated weights")
    ap.add_argument("--on-disk", metavar="CACHE_FILE",
                    help="the reference's second binary (qwen2_on_disk): one layer's weights and one K/V pair on the device, the "
                         "layers streamed from --weights every step and the KV cache kept in CACHE_FILE; same answers")
    a = ap.parse_args()
    from .qwen2 import ON_DISK, QWEN2_0_5B, Qwen2
    import dataclasses
    tok = Tokenizer.load(a.tokenizer)
    if a.on_disk:
        if not a.weights:
            ap.error("--on-disk needs --weights")
        model = Qwen2(dataclasses.replace(QWEN2_0_5B, max_seq=2048, flags=QWEN2_0_5B.flags | ON_DISK))
        model.open_files(a.weights, a.on_disk)
    else:
        model = Qwen2(dataclasses.replace(QWEN2_0_5B, seed=a.seed, max_seq=2048))
        if a.weights:
            from .convert import load_qwen2_flat
            load_qwen2_flat(model, a.weights)
    session = ChatSession(lambda t, p: int(model.infer([t], [p])[0]), tok, max_seq=2048)
    try:
        for line in sys.stdin.buffer:
            sys.stdout.buffer.write(session.turn(line.rstrip(b"\r\n")))
            sys.stdout.buffer.flush()
    finally:
        model.close()


if __name__ == "__main__":
    main()
