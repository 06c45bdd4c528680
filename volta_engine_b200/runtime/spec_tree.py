"""Token trees for speculative verification: several candidate continuations that share prefixes are verified in ONE
forward of the target model, and the longest branch the target agrees with is kept.

A tree is a list of nodes in topological order. Node 0 is the anchor (the last committed token, which has not been run
through the model yet); node i > 0 proposes ``tokens[i]`` as the token that follows its parent's. In the verify forward
  * node i is stored at cache position ``pos0 + i`` (every node has its own cache row),
  * its rotary position is ``pos0 + depth(i)`` (what it would be on a linear sequence),
  * its attention sees the prefix [0, pos0) and, inside the block, only its ancestors and itself (a 64-bit mask per row,
    read by the paged attention kernel),
so every node's logits equal those of the linear sequence prefix + path(i). Acceptance walks from the root: the target's
token at a node selects the child that proposed exactly that token. The accepted nodes' cache rows are then moved to
the consecutive positions pos0 + 1, pos0 + 2, ... (``PagedKVCache.move_rows``) and the sequence continues as if only the
accepted branch had been run.

The reference drafts linear chains only (src/runtime/mtp_runner.cpp:147-276, src/runtime/suffix_runner.cpp); there is no
tree attention mask in it. Sources of trees here: several earlier occurrences of the current suffix (``SuffixIndex``), or
a drafted chain with alternatives per position (a block drafter's candidate lists).
"""
from __future__ import annotations

from dataclasses import dataclass, field

MAX_NODES = 64


@dataclass
class TokenTree:
    tokens: list[int]
    parents: list[int] = field(default_factory=lambda: [-1])

    def __post_init__(self):
        assert len(self.tokens) == len(self.parents) and self.parents[0] == -1 and len(self.tokens) <= MAX_NODES
        assert all(0 <= p < i for i, p in enumerate(self.parents) if i), "nodes come after their parents"

    def __len__(self):
        return len(self.tokens)

    @property
    def depths(self) -> list[int]:
        d = [0] * len(self.tokens)
        for i in range(1, len(self.tokens)):
            d[i] = d[self.parents[i]] + 1
        return d

    @property
    def masks(self) -> list[int]:
        """Bit j of masks[i]: node j is node i or one of its ancestors."""
        m = [1] * len(self.tokens)
        for i in range(1, len(self.tokens)):
            m[i] = m[self.parents[i]] | (1 << i)
        return m

    def children(self, i: int) -> list[int]:
        return [j for j in range(i + 1, len(self.tokens)) if self.parents[j] == i]

    @classmethod
    def from_paths(cls, anchor: int, paths, max_nodes: int = MAX_NODES) -> "TokenTree":
        """Merge candidate continuations (token lists) into a trie under the anchor; earlier paths win the node budget."""
        tokens, parents = [anchor], [-1]
        kids: dict[tuple[int, int], int] = {}
        for path in paths:
            at = 0
            for t in path:
                nxt = kids.get((at, int(t)))
                if nxt is None:
                    if len(tokens) >= max_nodes:
                        break
                    nxt = len(tokens)
                    tokens.append(int(t))
                    parents.append(at)
                    kids[(at, int(t))] = nxt
                at = nxt
        return cls(tokens, parents)

    @classmethod
    def comb(cls, anchor: int, chain, alternatives, max_nodes: int = MAX_NODES) -> "TokenTree":
        """A drafted chain plus, per position, other candidates for that position (leaves beside the chain's node)."""
        paths = [list(chain)]
        for d, alts in enumerate(alternatives):
            for a in alts:
                if d < len(chain) and int(a) != int(chain[d]):
                    paths.append(list(chain[:d]) + [int(a)])
        return cls.from_paths(anchor, paths, max_nodes)

    def accept(self, targets) -> tuple[list[int], list[int]]:
        """``targets[i]``: the target model's token after node i. Returns (accepted node indices from the root down, the
        tokens to emit: the accepted proposals followed by the target's token at the last accepted node)."""
        path, at = [0], 0
        while True:
            want = int(targets[at])
            nxt = next((j for j in self.children(at) if self.tokens[j] == want), None)
            if nxt is None:
                break
            path.append(nxt)
            at = nxt
        return path, [self.tokens[i] for i in path[1:]] + [int(targets[at])]
