"""Two tiny configurations of the architecture that differ in every size and option,
the sequences the tests run, and the ways of cutting them into steps."""
from __future__ import annotations

import random
from typing import Dict, List, Tuple

import torch

TINY_A = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=64,
              num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=128, vocab_size=256,
              rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=512)
TINY_B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=3, hidden_size=96,
              num_attention_heads=6, num_key_value_heads=2, head_dim=32, intermediate_size=160, vocab_size=311,
              rope_theta=1e6, rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=1024)
TINY = {"A": (TINY_A, 0, 16), "B": (TINY_B, 1, 8)}        # config, weight seed, page size


def make_model_dir(path: str, which: str, store_dtype=torch.float32) -> str:
    from reinfer_b200.config import Qwen3Config
    from reinfer_b200.weights import write_random_model
    cfg, seed, _ = TINY[which]
    return write_random_model(path, Qwen3Config.from_dict(cfg), seed, store_dtype)


def sequences(which: str, lengths=None, seed=7) -> Dict[str, List[int]]:
    cfg = TINY[which][0]
    rnd = random.Random(seed)
    lengths = lengths or ([5, 17, 33, 70, 40, 26, 51] if which == "A" else [1, 9, 24, 50, 90, 37, 64, 12, 77, 58])
    return {f"r{i}": [rnd.randrange(cfg["vocab_size"]) for _ in range(n)] for i, n in enumerate(lengths)}


Step = Tuple[List[Tuple[str, List[int], List[int]]], List[str]]     # (entries (id, tokens, want), end)


def cut_whole(seqs) -> List[Step]:
    return [([(r, t, list(range(len(t))))], [r]) for r, t in seqs.items()]


def cut_tail_one_by_one(seqs, tail=32) -> List[Step]:
    steps: List[Step] = []
    for r, t in seqs.items():
        head = max(len(t) - tail, 0)
        if head:
            steps.append(([(r, t[:head], list(range(head)))], []))
        for i in range(head, len(t)):
            steps.append(([(r, [t[i]], [0])], [r] if i == len(t) - 1 else []))
    return steps


def cut_portions(seqs, sizes=(7, 2, 13, 3, 2, 5, 2, 11)) -> List[Step]:
    steps: List[Step] = []
    for r, t in seqs.items():
        i, k = 0, 0
        while i < len(t):
            n = min(sizes[k % len(sizes)], len(t) - i)
            k += 1
            steps.append(([(r, t[i:i + n], list(range(n)))], [r] if i + n == len(t) else []))
            i += n
    return steps


def cut_mixed(seqs, seed=3, max_live=4, decode_tail=12) -> List[Step]:
    """Up to `max_live` requests at a time; each brings portions of random size until its last
    `decode_tail` tokens, which come one by one beside the others' portions; a request may sit
    out a step; a finished request's pages are taken by the next."""
    rnd = random.Random(seed)
    waiting = list(seqs)
    live: Dict[str, int] = {}
    steps: List[Step] = []
    while waiting or live:
        while waiting and len(live) < max_live:
            live[waiting.pop(0)] = 0
        entries, end = [], []
        for r in list(live):
            if len(live) > 1 and rnd.random() < 0.2:
                continue                                           # sits this step out
            t, i = seqs[r], live[r]
            left = len(t) - i
            n = 1 if left <= decode_tail else min(rnd.choice([2, 3, 5, 8, 13]), left - decode_tail)
            entries.append((r, t[i:i + n], list(range(n))))
            live[r] = i + n
            if live[r] == len(t):
                end.append(r)
                del live[r]
        if entries:
            steps.append((entries, end))
    return steps


def pool_tokens_needed(steps: List[Step], page: int = 64) -> int:
    """Most tokens that live requests hold at once, each request's count rounded up to whole pages of `page`
    tokens: with page = the engine's page size this is exactly what the steps need and not a page more (so
    pages that a finished request gives back are the only ones a later request can get); with page = 64 it
    is the `--max-tokens` rule of bin/trace_run."""
    held: Dict[str, int] = {}
    worst = 0
    for entries, end in steps:
        for r, t, _ in entries:
            held[r] = held.get(r, 0) + len(t)
        worst = max(worst, sum(-(-n // page) * page for n in held.values()))
        for r in end:
            held.pop(r, None)
    return worst


class PageOwners:
    """Watches a cache manager between steps and counts the pages that passed from one request to another."""

    def __init__(self, cache, group: int = 0):
        self.cache, self.group = cache, group
        self.owner: Dict[int, str] = {}
        self.reused = set()

    def look(self) -> None:
        for rid in self.cache.live():
            for p in self.cache.table(rid, self.group):
                if p < 0:
                    continue
                if p in self.owner and self.owner[p] != rid:
                    self.reused.add(p)
                self.owner[p] = rid
