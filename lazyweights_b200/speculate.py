"""Greedy generation and prompt-lookup speculation on top of rt_forward.

Mirrors the reference CLI's `spec` mode (kernels/llmrt.cu:3024-3183): the draft is the continuation of the latest
earlier occurrence of the last `ngram` tokens (:3105-3112); one forward pass verifies [last token] + drafts (at most
eight tokens, the fused small-M product); the longest prefix on which the draft equals the greedy argmax is accepted and
the position is rewound to pos0 + 1 + accepted with rt_set_pos (:3144-3159).  The output equals plain greedy decoding
(up to float ties), because a verify pass reproduces the single-token logits.
"""
import numpy as np


def greedy(bundle, prompt, n_new, on_device=False):
    """Plain greedy decoding: returns the generated ids.  on_device: the tokens after the first are chosen by the
    runtime itself (rt_decode_greedy: no round trip per token); the ids are the same."""
    bundle.reset()
    tok = int(np.argmax(bundle.forward(np.asarray(prompt, np.int32))))
    out = [tok]
    if on_device and n_new > 1:
        return out + [int(t) for t in bundle.decode_greedy(tok, n_new - 1)]
    while len(out) < n_new:
        tok = int(np.argmax(bundle.forward(np.array([tok], np.int32))))
        out.append(tok)
    return out


def lookup_draft(history, ngram, n_draft):
    """Continuation of the latest earlier match of the last n tokens, for n = ngram down to 1: the first length that
    has a match decides (reference: kernels/llmrt.cu:3105-3112).  Empty if no length matches."""
    h = list(history)
    s = len(h)
    for n in range(min(ngram, s - 1), 0, -1):
        key = h[s - n:]
        for start in range(s - n - 1, -1, -1):
            if h[start:start + n] == key:
                d = h[start + n:start + n + n_draft]
                if d:
                    return d
                break                                    # the reference stops at the latest match of this length
    return []


class NgramCacheDrafter:
    """The n-gram cache drafter (the reference CLI's `--drafter ngramcache`, kernels/llmrt.cu:2604-2661; llama.cpp's
    prompt-lookup cache without static / dynamic files): n-grams (n = 1..4) of the prompt and every accepted token ->
    counts of the next token; each draft token comes from the longest n-gram whose most frequent continuation has
    enough samples and share.  The cache lives in the library's host code (lw_ngram_*)."""

    def __init__(self):
        from . import _native as nat
        self._nat = nat
        self._h = nat.lib().lw_ngram_create()
        self._n = 0

    def sync(self, history):
        """Feeds the tokens of `history` that the cache has not seen yet (one at a time, as the reference does)."""
        import ctypes as C
        new = np.ascontiguousarray(history[self._n:], np.int32)
        if new.size:
            self._nat.check(self._nat.lib().lw_ngram_push(C.c_void_p(self._h), new.ctypes.data_as(C.c_void_p), int(new.size)))
            self._n += int(new.size)

    def draft(self, history, n_draft):
        import ctypes as C
        self.sync(history)
        out = np.zeros(max(n_draft, 1), np.int32)
        n = self._nat.check(self._nat.lib().lw_ngram_draft(C.c_void_p(self._h), out.ctypes.data_as(C.c_void_p), int(n_draft)))
        return [int(t) for t in out[:n]]

    def close(self):
        if self._h:
            self._nat.lib().lw_ngram_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def prompt_lookup(bundle, prompt, n_new, n_draft=7, ngram=3, drafter="lookup"):
    """Greedy decoding with drafts from the plain prompt lookup (drafter="lookup") or from the n-gram cache
    (drafter="ngramcache"); returns (generated ids, forward passes, accepted drafts)."""
    cache = NgramCacheDrafter() if drafter == "ngramcache" else None
    bundle.reset()
    history = [int(t) for t in prompt]
    tok = int(np.argmax(bundle.forward(np.asarray(prompt, np.int32))))
    out, passes, accepted_total = [tok], 1, 0
    history.append(tok)
    while len(out) < n_new:
        room = min(n_draft, n_new - len(out))
        draft = cache.draft(history, room) if cache else lookup_draft(history, ngram, room)
        pos0 = bundle.pos
        logits = bundle.forward(np.array([tok] + draft, np.int32), all_logits=True)
        passes += 1
        choice = logits.argmax(1)
        accepted = 0
        while accepted < len(draft) and int(choice[accepted]) == draft[accepted]:
            accepted += 1
        new = draft[:accepted] + [int(choice[accepted])]
        bundle.set_pos(pos0 + 1 + accepted)      # drop the cache entries of rejected drafts
        accepted_total += accepted
        for t in new:
            if len(out) < n_new:
                out.append(t)
                history.append(t)
        tok = out[-1]
    return out, passes, accepted_total
