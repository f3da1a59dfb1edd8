"""The MTP speculative-decode loops of the reference drivers (engine/bench/spec27b.cpp:34-110) on top of an engine
object that exposes forward / accept / mtp_forward / topk (the CUDA engine or the CPU oracle model)."""
import numpy as np


def prefill(eng, prompt, slot=0, chunk=8, with_mtp=True, h_shift=None):
    """Target prefill in chunks of <= 8 rows (the verify path; the reference prefills token by token, spec27b.cpp:66-71)
    followed chunk by chunk by the MTP catch-up over the prompt: MTP at position p takes (token_p, h_target(p-1)),
    h_target(-1) = 0 (spec27b.cpp:62-64). h_shift(prev_last_row, T) must return the device pointer / host array of the
    T rows [h(p0-1), h(p0) .. h(p0+T-2)] for the engine at hand. Returns the position after the prompt."""
    pos = 0
    prev = None
    while pos < len(prompt):
        toks = prompt[pos:pos + chunk]
        eng.forward([(slot, toks, pos)])
        eng.accept(slot, len(toks))
        if with_mtp:
            h_in, prev = h_shift(prev, len(toks))
            eng.mtp_forward(slot, toks, h_in, pos)
        pos += len(toks)
    return pos


def plain_greedy(eng, first_pos, n_gen, slot=0):
    """T = 1 greedy stream (spec27b.cpp:34-40). The prompt must have been prefilled; returns n_gen tokens."""
    ids, _ = eng.topk(0, eng._last_T) if hasattr(eng, "_last_T") else eng.topk(0, 1)
    cur = int(ids[-1])
    out = []
    pos = first_pos
    for _ in range(n_gen):
        out.append(cur)
        eng.forward([(slot, [cur], pos)])
        eng.accept(slot, 1)
        pos += 1
        cur = int(eng.topk(0, 1)[0][0])
    return out


def seeded_substitutions(plain, emitted, n_draft, rate, rng, vocab):
    """Drafts for the next round: with probability `rate` the trunk's own next token (taken from the plain greedy stream),
    otherwise a token that is certainly different, so that the per-draft acceptance probability is exactly `rate`."""
    k = emitted - 1            # index in `plain` of the last emitted token
    sub = []
    for i in range(n_draft):
        good = plain[k + 1 + i]
        sub.append(good if rng.random() < rate else (good + 1) % vocab)
    return sub
