"""Evaluator: routes a trained model to the ranking protocol of its scoring technique and writes
``eval_report.json`` (reference ``dicee/evaluation/evaluator.py:32-722``).

* KvsAll / AllvsAll / 1vsAll / 1vsSample / KvsSample: tail-only filtered ranking over triples that already
  contain the reciprocal half (``:363-438``);
* NegSample: head and tail ranking through the triple path, metrics over ``2N`` (``:246-272``);
* byte-pair-encoded variants (``:274-361``);
* ``dummy_eval`` re-evaluates from the ``.npy`` splits of a stored run (``:645-679``).

The filter vocabularies are CSR arrays held by the :class:`KG`; the reference's pickled dictionaries
(``er_vocab.p`` …) are still written so existing tooling keeps working.
"""
from __future__ import annotations

import json
import os
import pickle
from typing import Dict, Optional

import numpy as np
import torch

from ..data.vocab import ee_csr, er_csr, re_csr
from .link_prediction import evaluate_bpe_lp, evaluate_lp_bpe_k_vs_all
from .ranking import head_and_tail_ranks, metrics_from_ranks, relation_ranks, tail_ranks


class Evaluator:
    def __init__(self, args, is_continual_training: bool = False):
        self.args = args
        self.is_continual_training = is_continual_training
        self.er_vocab = self.re_vocab = self.ee_vocab = None
        self.num_entities: Optional[int] = None
        self.num_relations: Optional[int] = None
        self.func_triple_to_bpe_representation = None
        self.domain_constraints_per_rel = None
        self.range_constraints_per_rel = None
        self.report: Dict = {}
        self.during_training = False
        self._pickles_written = False

    # ------------------------------------------------------------------ vocab
    def vocab_preparation(self, dataset) -> None:
        self.num_entities = dataset.num_entities
        self.num_relations = dataset.num_relations
        self.func_triple_to_bpe_representation = getattr(dataset, "func_triple_to_bpe_representation", None)
        if getattr(dataset, "er_csr", None) is not None:
            self.er_vocab, self.re_vocab = dataset.er_csr, dataset.re_csr
            self.ee_vocab = None
            self._dataset = dataset
        else:
            self.er_vocab, self.re_vocab, self.ee_vocab = dataset.er_vocab, dataset.re_vocab, dataset.ee_vocab
        path = getattr(self.args, "full_storage_path", None)
        if path and not self._pickles_written and not self.during_training and hasattr(dataset, "save_filter_vocab_pickles"):
            if (dataset.num_entities or 0) <= 2_000_000:  # dict export is a convenience for small graphs
                # a helper process writes them while the ranking runs; ``dataset.wait_for_vocab_pickles()`` joins it
                # (the executor does so before it returns, and the dataset does at interpreter exit)
                dataset.save_filter_vocab_pickles(path, background=True)
            self._pickles_written = True

    def _ee(self):
        if self.ee_vocab is None and getattr(self, "_dataset", None) is not None:
            self.ee_vocab = self._dataset.ee_csr
        return self.ee_vocab

    # ------------------------------------------------------------------ entry point
    def eval(self, dataset, trained_model, form_of_labelling: str, during_training: bool = False) -> Optional[Dict]:
        self.during_training = during_training
        if self.args.eval_model is None:
            return None
        self.vocab_preparation(dataset)
        if getattr(self.args, "num_folds_for_cv", 0) > 1:
            return None
        if isinstance(self.args.eval_model, bool):
            self.args.eval_model = "train_val_test"
        st, bpe = self.args.scoring_technique, getattr(self.args, "byte_pair_encoding", False)
        if st == "NegSample" and bpe:
            self.eval_rank_of_head_and_tail_byte_pair_encoded_entity(
                train_set=dataset.train_set, valid_set=dataset.valid_set, test_set=dataset.test_set,
                ordered_bpe_entities=dataset.ordered_bpe_entities, trained_model=trained_model)
        elif st in ("AllvsAll", "KvsAll", "1vsSample", "1vsAll") and bpe:
            if self.args.model != "BytE":
                self.eval_with_bpe_vs_all(raw_train_set=dataset.raw_train_set, raw_valid_set=dataset.raw_valid_set,
                                          raw_test_set=dataset.raw_test_set, trained_model=trained_model,
                                          form_of_labelling=form_of_labelling)
            else:
                self.eval_with_byte(raw_train_set=dataset.raw_train_set, raw_valid_set=dataset.raw_valid_set,
                                    raw_test_set=dataset.raw_test_set, trained_model=trained_model,
                                    form_of_labelling=form_of_labelling)
        elif st == "NegSample":
            self.eval_rank_of_head_and_tail_entity(train_set=dataset.train_set, valid_set=dataset.valid_set,
                                                   test_set=dataset.test_set, trained_model=trained_model)
        elif st in ("AllvsAll", "KvsAll", "1vsSample", "KvsSample", "1vsAll"):
            self.eval_with_vs_all(train_set=dataset.train_set, valid_set=dataset.valid_set,
                                  test_set=dataset.test_set, trained_model=trained_model,
                                  form_of_labelling=form_of_labelling)
        else:
            raise ValueError(f"Invalid scoring technique: {st}")
        if not self.during_training:
            with open(os.path.join(self.args.full_storage_path, "eval_report.json"), "w") as f:
                json.dump(self.report, f, indent=4)
        return dict(self.report)

    def _splits(self, train_set, valid_set, test_set, which: Optional[str] = None):
        which = which if which is not None else self.args.eval_model
        if "train" in which:
            yield "Train", train_set
        if "val" in which and valid_set is not None:
            yield "Val", valid_set
        if "test" in which and test_set is not None:
            yield "Test", test_set

    # ------------------------------------------------------------------ protocols
    def eval_with_vs_all(self, *, train_set, valid_set=None, test_set=None, trained_model, form_of_labelling,
                         which: Optional[str] = None) -> None:
        for name, split in self._splits(train_set, valid_set, test_set, which):
            self.report[name] = self.evaluate_lp_k_vs_all(trained_model, split,
                                                          f"Evaluate {trained_model.name} on {name} set",
                                                          form_of_labelling)

    def evaluate_lp_k_vs_all(self, model, triple_idx, info: Optional[str] = None,
                             form_of_labelling: Optional[str] = None) -> Dict[str, float]:
        model.eval()
        bs = max(int(getattr(self.args, "batch_size", 1024) or 1024), 1)
        if form_of_labelling == "RelationPrediction":
            ranks = relation_ranks(model, triple_idx, self._ee(), bs)
        else:
            fused = False if getattr(self.args, "kernel_backend", "auto") == "torch" else None
            ranks = tail_ranks(model, triple_idx, self.er_vocab, bs, fused=fused)
        assert ranks.numel() == len(triple_idx)
        res = metrics_from_ranks(ranks, divisor=len(triple_idx))
        if info and not self.during_training:
            print(info)
            print(res)
        return res

    def eval_rank_of_head_and_tail_entity(self, *, train_set, valid_set=None, test_set=None, trained_model,
                                          which: Optional[str] = None) -> None:
        for name, split in self._splits(train_set, valid_set, test_set, which):
            self.report[name] = self.evaluate_lp(trained_model, split, f"Evaluate {trained_model.name} on {name} set")

    def evaluate_lp(self, model, triple_idx, info: str) -> Dict[str, float]:
        model.eval()
        hr, tr = head_and_tail_ranks(model, triple_idx, self.num_entities, self.er_vocab, self.re_vocab,
                                     batch_size=128, chunk_size=1000)
        res = metrics_from_ranks(torch.cat((hr, tr)), divisor=2 * len(triple_idx))
        if info and not self.during_training:
            print(info)
            print(res)
        return res

    def eval_rank_of_head_and_tail_byte_pair_encoded_entity(self, *, train_set=None, valid_set=None, test_set=None,
                                                            ordered_bpe_entities, trained_model) -> None:
        for name, split in self._splits(train_set, valid_set, test_set):
            rows = [tuple(tuple(int(v) for v in part) for part in tr) for tr in np.asarray(split).tolist()]
            self.report[name] = evaluate_bpe_lp(trained_model, rows, ordered_bpe_entities, self.er_vocab,
                                                self.re_vocab, info=f"Evaluate {trained_model.name} on {name}")

    def eval_with_bpe_vs_all(self, *, raw_train_set, raw_valid_set=None, raw_test_set=None, trained_model,
                             form_of_labelling) -> None:
        str_idx = {s: i for i, (s, _, _) in enumerate(trained_model.args["ordered_bpe_entities"])}
        er: Dict = {}
        for df in (raw_train_set, raw_valid_set, raw_test_set):
            if df is not None:
                for h, r, t in df.values.tolist():
                    er.setdefault((h, r), []).append(t)
        for name, df in self._splits(raw_train_set, raw_valid_set, raw_test_set):
            self.report[name] = evaluate_lp_bpe_k_vs_all(
                trained_model, df.values.tolist(), er_vocab=er, batch_size=self.args.batch_size,
                func_triple_to_bpe_representation=self.func_triple_to_bpe_representation,
                str_to_bpe_entity_to_idx=str_idx)

    @torch.no_grad()
    def eval_with_byte(self, *, raw_train_set, raw_valid_set=None, raw_test_set=None, trained_model,
                       form_of_labelling) -> None:
        """BytE: teacher-forced next-token accuracy and perplexity over the ``h r t.`` token stream of each
        split (the reference's generative evaluation, ``evaluator.py:305-329,513-552``, only prints samples)."""
        from ..data.bpe import get_tokenizer
        enc = get_tokenizer()
        bs = trained_model.config.block_size
        space, end = enc.encode(" ")[0], enc.encode(".")[0]
        trained_model.eval()
        dev = trained_model.device
        for name, df in self._splits(raw_train_set, raw_valid_set, raw_test_set):
            stream = []
            for h, r, t in df.values.tolist()[:2000]:
                stream.extend([*enc.encode(str(h)), space, *enc.encode(str(r)), space, *enc.encode(str(t)), end])
            tok = torch.tensor(stream, dtype=torch.long)
            if tok.numel() <= bs:
                continue
            win = tok.unfold(0, bs + 1, bs)
            x, y = win[:, :-1].to(dev), win[:, 1:].to(dev)
            logits = trained_model(x)
            loss = torch.nn.functional.cross_entropy(logits.reshape(-1, logits.size(-1)), y.reshape(-1))
            acc = (logits.argmax(-1) == y).float().mean()
            self.report[name] = {"NextTokenAcc": float(acc), "Perplexity": float(torch.exp(loss))}

    # ------------------------------------------------------------------ stored runs
    def _load_indexed_datasets(self):
        p = self.args.full_storage_path
        def ld(n):
            f = os.path.join(p, n)
            return np.load(f) if os.path.isfile(f) else None
        return ld("train_set.npy"), ld("valid_set.npy"), ld("test_set.npy")

    def dummy_eval(self, trained_model, form_of_labelling: str) -> None:
        """Evaluate from the artefacts of a stored run directory (continual training)."""
        assert trained_model is not None
        if self.args.eval_model is None:
            return
        p = self.args.full_storage_path
        train, valid, test = self._load_indexed_datasets()
        self.num_entities = getattr(self.args, "num_entities", None)
        self.num_relations = getattr(self.args, "num_relations", None)
        data = np.concatenate([s for s in (train, valid, test) if s is not None]).astype(np.int64) \
            if (valid is not None and test is not None) else train.astype(np.int64)
        if self.num_entities is None:
            self.num_entities = int(data[:, [0, 2]].max()) + 1
            self.num_relations = int(data[:, 1].max()) + 1
        self.er_vocab = er_csr(data, self.num_relations)
        self.re_vocab = re_csr(data, self.num_entities)
        self.ee_vocab = ee_csr(data, self.num_entities)
        if self.args.scoring_technique == "NegSample":
            self.eval_rank_of_head_and_tail_entity(train_set=train, valid_set=valid, test_set=test,
                                                   trained_model=trained_model)
        else:
            self.eval_with_vs_all(train_set=train, valid_set=valid, test_set=test, trained_model=trained_model,
                                  form_of_labelling=form_of_labelling)
        with open(os.path.join(p, "eval_report.json"), "w") as f:
            json.dump(self.report, f, indent=4)

    def eval_with_data(self, dataset, trained_model, triple_idx: np.ndarray, form_of_labelling: str) -> Dict:
        """Evaluate on explicitly given index triples."""
        self.vocab_preparation(dataset)
        if self.args.scoring_technique == "NegSample":
            return self.evaluate_lp(trained_model, triple_idx, "Evaluate on given data")
        return self.evaluate_lp_k_vs_all(trained_model, triple_idx, "Evaluate on given data", form_of_labelling)
