"""Sampling of multi-hop (EPFO + negation) queries with easy and hard answers.

Covers the fourteen query structures of the reference (``dicee/query_generator.py:32-46``): 1p 2p 3p 2i 3i ip pi
2in 3in inp pin pni 2u up.  A query is a nested tuple in the notation the interactive API accepts
(``KGE.answer_multi_hop_query``): ``(anchor, (r1, r2, ...))`` for paths, tuples of those for intersections, a
trailing ``('u',)`` for unions, ``'n'`` after a relation for negation of that branch.

Queries are grounded *backwards*: an answer entity is drawn, then every branch is filled by walking incoming
edges of the larger graph (train+valid(+test)) until an anchor is reached.  Answers are computed *forwards* by set
traversal; answers reachable in the smaller graph are "easy", the rest "hard" (they need the held-out edges).
"""
from __future__ import annotations

import os
import pickle
import random
from collections import defaultdict
from typing import Dict, List, Set, Tuple

QUERY_STRUCTS = {
    "1p": ("e", ("r",)), "2p": ("e", ("r", "r")), "3p": ("e", ("r", "r", "r")),
    "2i": (("e", ("r",)), ("e", ("r",))), "3i": (("e", ("r",)), ("e", ("r",)), ("e", ("r",))),
    "pi": (("e", ("r", "r")), ("e", ("r",))), "ip": ((("e", ("r",)), ("e", ("r",))), ("r",)),
    "2in": (("e", ("r",)), ("e", ("r", "n"))), "3in": (("e", ("r",)), ("e", ("r",)), ("e", ("r", "n"))),
    "pin": (("e", ("r", "r")), ("e", ("r", "n"))), "pni": (("e", ("r", "r", "n")), ("e", ("r",))),
    "inp": ((("e", ("r",)), ("e", ("r", "n"))), ("r",)),
    "2u": (("e", ("r",)), ("e", ("r",)), ("u",)), "up": ((("e", ("r",)), ("e", ("r",)), ("u",)), ("r",)),
}


def _is_path(s) -> bool:
    """``(head, (op, op, ...))``: the second element is a flat tuple of relations / ``'n'`` markers."""
    return (len(s) == 2 and isinstance(s[1], tuple) and s[1] != ("u",)
            and all(not isinstance(o, tuple) for o in s[1]))


class Graph:
    """Adjacency as ``out[h][r] -> {t}`` and ``inc[t][r] -> {h}`` over integer ids."""

    def __init__(self, num_entities: int):
        self.num_entities = num_entities
        self.out: Dict[int, Dict[int, Set[int]]] = defaultdict(lambda: defaultdict(set))
        self.inc: Dict[int, Dict[int, Set[int]]] = defaultdict(lambda: defaultdict(set))

    def add(self, triples) -> "Graph":
        for h, r, t in triples:
            self.out[h][r].add(t)
            self.inc[t][r].add(h)
        return self


class QueryGenerator:
    def __init__(self, train_path: str, val_path: str, test_path: str, ent2id: Dict = None, rel2id: Dict = None,
                 seed: int = 1, gen_valid: bool = False, gen_test: bool = True):
        self.train_path, self.val_path, self.test_path = train_path, val_path, test_path
        self.gen_valid, self.gen_test = gen_valid, gen_test
        self.ent2id, self.rel2id = ent2id, rel2id
        self.seed = seed
        self.max_ans_num = 1e6
        self.query_name_to_struct = dict(QUERY_STRUCTS)
        self.set_global_seed(seed)
        self._graphs = None

    def set_global_seed(self, seed: int) -> None:
        self.rng = random.Random(seed)

    # ------------------------------------------------------------------ graphs
    def _read(self, path: str) -> List[Tuple[int, int, int]]:
        rows = []
        if path is None or not os.path.isfile(path):
            return rows
        with open(path) as f:
            for line in f:
                p = line.split()
                if len(p) < 3:
                    continue
                h, r, t = p[0], p[1], p[2]
                if self.ent2id is not None:
                    if h not in self.ent2id or t not in self.ent2id or r not in self.rel2id:
                        continue
                    rows.append((self.ent2id[h], self.rel2id[r], self.ent2id[t]))
                else:
                    rows.append((int(h), int(r), int(t)))
        return rows

    def construct_graph(self, paths: List[str]) -> Graph:
        n = len(self.ent2id) if self.ent2id is not None else 0
        g = Graph(n)
        for p in paths:
            g.add(self._read(p))
        if not n:
            g.num_entities = 1 + max(list(g.out.keys()) + list(g.inc.keys()) + [0])
        return g

    def _get_graphs(self) -> Tuple[Graph, Graph]:
        """(small graph for easy answers, full graph for grounding and hard answers)."""
        if self._graphs is None:
            if self.gen_test:
                small = self.construct_graph([self.train_path, self.val_path])
                full = self.construct_graph([self.train_path, self.val_path, self.test_path])
            elif self.gen_valid:
                small = self.construct_graph([self.train_path])
                full = self.construct_graph([self.train_path, self.val_path])
            else:
                small = full = self.construct_graph([self.train_path])
            self._graphs = (small, full)
        return self._graphs

    # ------------------------------------------------------------------ grounding (backward)
    def _fill(self, struct, answer: int, g: Graph):
        """Return the grounded structure or ``None`` when the walk dead-ends."""
        if _is_path(struct):
            ops = list(struct[1])
            cur = answer
            last_r = None
            for i in range(len(ops) - 1, -1, -1):
                if ops[i] == "n":
                    continue
                cand = list(g.inc[cur].keys()) if cur in g.inc else []
                if last_r is not None:  # avoid walking straight back over the inverse of the previous relation
                    cand = [r for r in cand if r // 2 != last_r // 2 or r == last_r] or cand
                if not cand:
                    return None
                r = self.rng.choice(cand)
                ops[i] = r
                last_r = r
                cur = self.rng.choice(sorted(g.inc[cur][r]))
            head = cur if struct[0] == "e" else self._fill(struct[0], cur, g)
            return None if head is None else (head, tuple(ops))
        parts = []
        for s in struct:
            if s == ("u",):
                parts.append(s)
                continue
            f = self._fill(s, answer, g)
            if f is None:
                return None
            parts.append(f)
        real = [p for p in parts if p != ("u",)]
        if len(set(real)) < len(real):
            return None  # identical branches make the query degenerate
        return tuple(parts)

    # ------------------------------------------------------------------ answering (forward)
    def achieve_answer(self, query, g: Graph) -> Set[int]:
        if _is_path(query):
            ents = {query[0]} if not isinstance(query[0], tuple) else self.achieve_answer(query[0], g)
            for op in query[1]:
                if op == "n":
                    ents = set(range(g.num_entities)) - ents
                else:
                    nxt: Set[int] = set()
                    for e in ents:
                        if e in g.out and op in g.out[e]:
                            nxt |= g.out[e][op]
                    ents = nxt
            return ents
        union = query[-1] == ("u",)
        branches = [q for q in query if q != ("u",)]
        ents = self.achieve_answer(branches[0], g)
        for b in branches[1:]:
            a = self.achieve_answer(b, g)
            ents = ents | a if union else ents & a
        return ents

    def ground_queries(self, query_structure, gen_num: int, query_name: str = ""):
        """Sample ``gen_num`` queries: returns ``(queries, tp_answers, fp_answers, fn_answers)`` keyed by query."""
        small, full = self._get_graphs()
        queries, tp, fp, fn = set(), {}, {}, {}
        ents = sorted(full.inc.keys())
        tries = 0
        while len(queries) < gen_num and tries < gen_num * 200 and ents:
            tries += 1
            q = self._fill(query_structure, self.rng.choice(ents), full)
            if q is None or q in queries:
                continue
            ans_full = self.achieve_answer(q, full)
            ans_small = self.achieve_answer(q, small)
            hard = ans_full - ans_small
            if not ans_full or len(ans_full) > self.max_ans_num:
                continue
            if (self.gen_test or self.gen_valid) and not hard:
                continue  # a held-out query must need held-out edges
            queries.add(q)
            tp[q] = ans_full & ans_small
            fp[q] = ans_small - ans_full
            fn[q] = hard
        return queries, tp, fp, fn

    def generate_queries(self, query_struct, gen_num: int, query_type: str):
        return self.ground_queries(query_struct, gen_num, query_type)

    def get_queries(self, query_type: str, gen_num: int):
        """Queries of one type with ids mapped back to strings when vocabularies were given."""
        qs, tp, fp, fn = self.ground_queries(self.query_name_to_struct[query_type], gen_num, query_type)
        return self.unmap(query_type, qs, tp, fp, fn)

    # ------------------------------------------------------------------ id <-> string
    def unmap_query(self, query, id2ent, id2rel):
        if _is_path(query):
            head = id2ent[query[0]] if not isinstance(query[0], tuple) else self.unmap_query(query[0], id2ent, id2rel)
            return (head, tuple(o if o == "n" else id2rel[o] for o in query[1]))
        return tuple(q if q == ("u",) else self.unmap_query(q, id2ent, id2rel) for q in query)

    def unmap(self, query_type, queries, tp_answers, fp_answers, fn_answers):
        if self.ent2id is None:
            return queries, tp_answers, fp_answers, fn_answers
        id2ent = {v: k for k, v in self.ent2id.items()}
        id2rel = {v: k for k, v in self.rel2id.items()}
        out_q, out_tp, out_fp, out_fn = [], {}, {}, {}
        for q in queries:
            s = self.unmap_query(q, id2ent, id2rel)
            out_q.append(s)
            out_tp[s] = {id2ent[e] for e in tp_answers[q]}
            out_fp[s] = {id2ent[e] for e in fp_answers[q]}
            out_fn[s] = {id2ent[e] for e in fn_answers[q]}
        return out_q, out_tp, out_fp, out_fn

    # ------------------------------------------------------------------ persistence
    def save_queries(self, query_type: str, gen_num: int, save_path: str) -> None:
        os.makedirs(save_path, exist_ok=True)
        data = self.get_queries(query_type, gen_num)
        with open(os.path.join(save_path, f"{query_type}_queries.pkl"), "wb") as f:
            pickle.dump(data, f)

    @staticmethod
    def load_queries(path: str):
        with open(path, "rb") as f:
            return pickle.load(f)

    @staticmethod
    def save_queries_and_answers(path: str, data) -> None:
        with open(path, "wb") as f:
            pickle.dump(data, f)

    @staticmethod
    def load_queries_and_answers(path: str):
        with open(path, "rb") as f:
            return pickle.load(f)
