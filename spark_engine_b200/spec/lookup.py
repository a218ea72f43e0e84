"""Prompt-lookup ("copy") drafts: if the last n tokens occurred earlier in the sequence, propose what followed.
Reference: engine-rs/src/qwen/lookup.rs (n = 3), spec_probe.rs copy_proposal."""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple


class LookupIndex:
    def __init__(self, n: int = 3):
        self.n = n
        self.tokens: List[int] = []
        self.last: Dict[Tuple[int, ...], int] = {}     # n-gram -> index just after its latest occurrence

    def extend(self, toks: Sequence[int]) -> None:
        for t in toks:
            self.tokens.append(int(t))
            if len(self.tokens) >= self.n:
                key = tuple(self.tokens[-self.n:])
                self.last[key] = len(self.tokens)

    def propose(self, depth: int) -> List[int]:
        """Continuation of the most recent EARLIER occurrence of the current n-gram suffix (may be empty)."""
        if len(self.tokens) < self.n:
            return []
        key = tuple(self.tokens[-self.n:])
        best = -1
        # the latest occurrence is the suffix itself: scan for the previous one
        for i in range(len(self.tokens) - self.n - 1, -1, -1):
            if tuple(self.tokens[i: i + self.n]) == key:
                best = i + self.n
                break
        if best < 0:
            return []
        return self.tokens[best: best + depth]
