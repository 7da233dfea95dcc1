"""Greedy generation and prompt-lookup speculation on top of rt_forward.

Mirrors the reference CLI's `spec` mode (kernels/llmrt.cu:3024-3183): the draft is the continuation of the latest
earlier occurrence of the last `ngram` tokens (:3105-3112); one forward pass verifies [last token] + drafts (at most
eight tokens, the fused small-M product); the longest prefix on which the draft equals the greedy argmax is accepted and
the position is rewound to pos0 + 1 + accepted with rt_set_pos (:3144-3159).  The output equals plain greedy decoding
(up to float ties), because a verify pass reproduces the single-token logits.
"""
import numpy as np


def greedy(bundle, prompt, n_new):
    """Plain greedy decoding: returns the generated ids."""
    bundle.reset()
    tok = int(np.argmax(bundle.forward(np.asarray(prompt, np.int32))))
    out = [tok]
    while len(out) < n_new:
        tok = int(np.argmax(bundle.forward(np.array([tok], np.int32))))
        out.append(tok)
    return out


def lookup_draft(history, ngram, n_draft):
    """Continuation of the latest earlier match of the last `ngram` tokens (empty if there is none)."""
    h = list(history)
    if len(h) <= ngram:
        return []
    key = h[-ngram:]
    for start in range(len(h) - ngram - 1, -1, -1):
        if h[start:start + ngram] == key:
            return h[start + ngram:start + ngram + n_draft]
    return []


def prompt_lookup(bundle, prompt, n_new, n_draft=7, ngram=3):
    """Greedy decoding with prompt-lookup drafts; returns (generated ids, forward passes, accepted drafts)."""
    bundle.reset()
    history = [int(t) for t in prompt]
    tok = int(np.argmax(bundle.forward(np.asarray(prompt, np.int32))))
    out, passes, accepted_total = [tok], 1, 0
    history.append(tok)
    while len(out) < n_new:
        draft = lookup_draft(history, ngram, min(n_draft, n_new - len(out)))
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
