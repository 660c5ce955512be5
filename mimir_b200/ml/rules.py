"""Association rules (reference: rules/rules.go): item sets that appear in at least ``min_support`` of
the baskets, found level by level (a candidate is counted only when every subset one item smaller is
frequent), and the rules ``if -> then`` among them with at least ``min_confidence``."""
from __future__ import annotations

import itertools
from dataclasses import dataclass


@dataclass
class Rule:
    if_: tuple          # the items a basket holds
    then: tuple         # the items it then tends to hold too
    support: float      # the share of baskets with all of them
    confidence: float   # of the baskets with ``if_``, the share that also hold ``then``
    lift: float         # confidence over the share of baskets with ``then``: above 1 means they go together


def mine(baskets, min_support: float = 0.01, min_confidence: float = 0.5, max_items: int = 3, top: int = 0) -> list:
    """The rules of ``baskets`` (lists of item names) by falling lift, then support; ``top`` keeps only the
    first n."""
    if not (0 < min_support <= 1) or not (0 <= min_confidence <= 1) or max_items < 2 or top < 0:
        raise ValueError("rules: support in (0, 1], confidence in [0, 1], at least two items per rule")
    sets = [frozenset(b) for b in baskets]
    n = len(sets)
    if n == 0:
        raise ValueError("rules: no baskets")
    need = min_support * n
    count: dict = {}
    for b in sets:
        for x in b:
            k = (x,)
            count[k] = count.get(k, 0) + 1
    frequent = {k: c for k, c in count.items() if c >= need}
    support = dict(frequent)
    level = sorted(frequent)
    size = 1
    while level and size < max_items:
        size += 1
        cands = set()
        for a, b in itertools.combinations(level, 2):
            if a[:-1] == b[:-1]:
                c = tuple(sorted(set(a) | set(b), key=str))
                if len(c) == size and all(tuple(s) in frequent for s in itertools.combinations(c, size - 1)):
                    cands.add(c)
        count = {c: 0 for c in cands}
        members = {c: frozenset(c) for c in cands}
        for b in sets:
            if len(b) < size:
                continue
            for c, fs in members.items():
                if fs <= b:
                    count[c] += 1
        frequent = {c: v for c, v in count.items() if v >= need}
        support.update(frequent)
        level = sorted(frequent, key=lambda t: tuple(map(str, t)))
    out = []
    for items, cnt in support.items():
        if len(items) < 2:
            continue
        for r in range(1, len(items)):
            for ante in itertools.combinations(items, r):
                cons = tuple(x for x in items if x not in ante)
                conf = cnt / support[tuple(ante)]
                if conf >= min_confidence:
                    out.append(Rule(tuple(ante), cons, cnt / n, conf, conf / (support[cons] / n)))
    out.sort(key=lambda r: (-r.lift, -r.support, tuple(map(str, r.if_)), tuple(map(str, r.then))))
    return out[:top] if top else out
