"""Model-free drafting from the sequence's own history: the continuation that followed the most recent
earlier occurrence of the current k-gram (reference: inc/engine/runtime/suffix_index.h:9-66,
src/runtime/suffix_runner.cpp)."""
from __future__ import annotations


class SuffixIndex:
    def __init__(self, max_k: int = 8, min_k: int = 2):
        self.max_k, self.min_k = max_k, min_k
        self.toks: list[int] = []
        self.last: dict[tuple, int] = {}   # k-gram -> index just after its latest occurrence

    def extend(self, toks) -> None:
        for t in toks:
            self.push(t)

    def push(self, tok: int) -> None:
        self.toks.append(tok)
        n = len(self.toks)
        for k in range(self.min_k, self.max_k + 1):
            if n - 1 >= k:   # the gram that ended one token ago now has a known continuation
                self.last[tuple(self.toks[n - 1 - k:n - 1])] = n - 1

    def draft(self, depth: int) -> list[int]:
        """Up to ``depth`` tokens that followed the latest earlier occurrence of the longest matching suffix."""
        n = len(self.toks)
        for k in range(min(self.max_k, n), self.min_k - 1, -1):
            pos = self.last.get(tuple(self.toks[n - k:]))
            if pos is not None and pos < n:
                return self.toks[pos:pos + depth]
        return []

    def truncate(self, n: int) -> None:
        """Roll back to the first n tokens (rejected drafts are never pushed, so this is only for rewinds)."""
        if n < len(self.toks):
            toks = self.toks[:n]
            self.toks, self.last = [], {}
            self.extend(toks)
