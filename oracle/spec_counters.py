"""Checker for the speculation driver: what the counters of a request must be, given only the tokens it emitted.

Test infrastructure (never imported by the product).  A restatement of the reference's own protocol oracle
(NomenAK/FlintNSteel tests/speed_native_smoke.py:41-98) and of the width policy of its driver
(tools/fns_serve/fns_serve.cpp:430-459), in this repository's words.
"""
from __future__ import annotations

COUNTERS = ("decode_iterations", "spec_windows", "spec_drafted", "spec_accepted", "spec_emitted")


def lookup_draft(history, want):
    """Prompt-lookup draft (tests/speed_native_smoke.py:41-47, include/fns/lookup.h:12-27): the ids that followed the
    latest earlier occurrence of the final n-gram, n = 4, 3, 2."""
    history = list(history)
    if want <= 0:
        return []
    for n in (4, 3, 2):
        if len(history) < n + 1:
            continue
        tail = history[-n:]
        for start in range(len(history) - n - 1, -1, -1):
            if history[start:start + n] == tail:
                return history[start + n:start + n + want]
    return []


def expected_counters(prompt, output, width, budget=None):
    """Counters and window list implied by the emitted ids alone (tests/speed_native_smoke.py:50-98, no grammar):
    every lookup's draft is submitted whole; choices are committed along the draft until a mismatch, the bonus column,
    the output budget or the end; drafted ids that were never emitted still count as drafted."""
    counts = dict.fromkeys(COUNTERS, 0)
    windows = []
    output = list(output)
    assert output, "no output"
    if width == 0:
        counts["decode_iterations"] = len(output) - 1
        return counts, windows
    history = list(prompt) + output[:1]
    budget = len(output) if budget is None else budget
    pos = 1
    while pos < len(output):
        counts["decode_iterations"] += 1
        draft = lookup_draft(history, min(width - 1, budget - pos))
        if not draft:
            history.append(output[pos])
            pos += 1
            continue
        counts["spec_windows"] += 1
        counts["spec_drafted"] += len(draft)
        start, accepted = pos, 0
        for column in range(len(draft) + 1):
            if pos == len(output):
                break
            token = output[pos]
            history.append(token)
            pos += 1
            counts["spec_emitted"] += 1
            if column == len(draft) or token != draft[column]:
                break
            accepted += 1
            counts["spec_accepted"] += 1
        windows.append({"start": start, "end": pos, "drafted": len(draft), "accepted": accepted})
    return counts, windows


def choose_width(cost, spec, accepted, offered, skipped_proposals, nd_max):
    """The adaptive width of tools/fns_serve/fns_serve.cpp:430-459: (draft ids to verify, new skipped_proposals)."""
    a = (accepted + 1) / (offered + 2)
    t1 = cost[1]
    if t1 == 0.0:
        for w in range(2, spec + 1):
            if cost[w] > 0.0:
                t1 = cost[w] / (1.0 + 0.25 * (w - 1))
                break
        if t1 == 0.0:
            t1 = 1.0
    best, best_score, expected, power = 0, 1.0, 1.0, 1.0
    for n in range(1, nd_max + 1):
        power *= a
        expected += power
        c = cost[n + 1] / t1 if cost[n + 1] > 0.0 else 1.0 + 0.25 * n
        if expected / c > best_score:
            best_score, best = expected / c, n
    if best == 0 and skipped_proposals >= 16:
        best = 1
    return best, (skipped_proposals + 1 if best == 0 else 0)
