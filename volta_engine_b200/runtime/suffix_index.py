"""Model-free drafting from the sequence's own history: the continuation that followed the most recent
earlier occurrence of the current k-gram (reference: inc/engine/runtime/suffix_index.h:9-66,
src/runtime/suffix_runner.cpp)."""
from __future__ import annotations


class SuffixIndex:
    def __init__(self, max_k: int = 8, min_k: int = 2):
        self.max_k, self.min_k = max_k, min_k
        self.toks: list[int] = []
        self.last: dict[tuple, int] = {}   # k-gram -> index just after its latest occurrence
        self.occ: dict[tuple, list[int]] = {}   # k-gram -> indices just after its latest occurrences (newest last)
        self.max_occ = 4

    def extend(self, toks) -> None:
        for t in toks:
            self.push(t)

    def push(self, tok: int) -> None:
        self.toks.append(tok)
        n = len(self.toks)
        for k in range(self.min_k, self.max_k + 1):
            if n - 1 >= k:   # the gram that ended one token ago now has a known continuation
                gram = tuple(self.toks[n - 1 - k:n - 1])
                self.last[gram] = n - 1
                lst = self.occ.setdefault(gram, [])
                lst.append(n - 1)
                if len(lst) > self.max_occ:
                    del lst[0]

    def draft(self, depth: int) -> list[int]:
        """Up to ``depth`` tokens that followed the latest earlier occurrence of the longest matching suffix."""
        n = len(self.toks)
        for k in range(min(self.max_k, n), self.min_k - 1, -1):
            pos = self.last.get(tuple(self.toks[n - k:]))
            if pos is not None and pos < n:
                return self.toks[pos:pos + depth]
        return []

    def draft_paths(self, depth: int, width: int) -> list[list[int]]:
        """Up to ``width`` different continuations (each up to ``depth`` tokens) for a verification tree: what followed the
        latest occurrences of the longest matching suffix, newest first, then those of shorter suffixes; continuations
        that start with a token already proposed are merged by the tree builder, so only new first tokens count."""
        n = len(self.toks)
        paths, firsts = [], set()
        for k in range(min(self.max_k, n), self.min_k - 1, -1):
            for pos in reversed(self.occ.get(tuple(self.toks[n - k:]), [])):
                if pos >= n:
                    continue
                cont = self.toks[pos:pos + depth]
                if cont and cont[0] not in firsts:
                    firsts.add(cont[0])
                    paths.append(cont)
                    if len(paths) >= width:
                        return paths
        return paths

    def truncate(self, n: int) -> None:
        """Roll back to the first n tokens (rejected drafts are never pushed, so this is only for rewinds)."""
        if n < len(self.toks):
            toks = self.toks[:n]
            self.toks, self.last, self.occ = [], {}, {}
            self.extend(toks)
