"""Association rules (reference: rules/rules.go): item sets that appear in at least ``min_support`` of
the baskets, found level by level (a candidate is counted only when every subset one item smaller is
frequent), and the rules ``if -> then`` among them with at least ``min_confidence``."""
from __future__ import annotations

import itertools
from dataclasses import dataclass

import torch


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
    level = sorted(frequent, key=lambda t: tuple(map(str, t)))
    # the baskets as a 0 / 1 table over the frequent items: the baskets that hold a set are counted by matrix
    # products (the columns of a set's first items multiplied together, times the table), not basket by basket
    column = {k[0]: j for j, k in enumerate(level)}
    table = torch.zeros(n, max(len(level), 1))
    held = [(r, column[x]) for r, b in enumerate(sets) for x in b if x in column]
    if held:
        at = torch.tensor(held, dtype=torch.long)
        table[at[:, 0], at[:, 1]] = 1.0
    size = 1
    while level and size < max_items:
        size += 1
        # candidates: two frequent sets that share all but their last item, every smaller subset frequent
        groups: dict = {}
        for c in level:
            groups.setdefault(c[:-1], []).append(c[-1])
        cands = []
        for prefix, lasts in groups.items():
            for x, y in itertools.combinations(lasts, 2):
                c = prefix + (x, y)
                if size == 2 or all(tuple(sub) in frequent for sub in itertools.combinations(c, size - 1)):
                    cands.append(c)
        count = {}
        by_prefix: dict = {}
        for c in cands:
            by_prefix.setdefault(c[:-1], []).append(c[-1])
        prefixes = list(by_prefix)
        for p0 in range(0, len(prefixes), 1024):
            part = prefixes[p0: p0 + 1024]
            cols = torch.tensor([[column[x] for x in pre] for pre in part], dtype=torch.long)       # [prefixes, size - 1]
            both = table[:, cols[:, 0]]
            for j in range(1, size - 1):
                both = both * table[:, cols[:, j]]
            counts = both.t() @ table                                                              # [prefixes, items]
            for r, pre in enumerate(part):
                row = counts[r]
                for last in by_prefix[pre]:
                    count[pre + (last,)] = int(round(float(row[column[last]])))
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
