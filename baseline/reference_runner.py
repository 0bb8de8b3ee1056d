"""Runs the *unmodified* reference (installed under ``baseline/_ref``) through its own public API
(``dicee.Execute(args).start()``) on the benchmark configurations and times K training steps.

Nothing of this repository's models, kernels or engine is on that path.  Three things are added around the
reference, none of which changes its code:

* import stand-ins for packages that are absent on the benchmark machines (``lightning``, ``pytorch_lightning``,
  ``polars``; see ``baseline/shims``) and a local byte tokenizer returned by ``tiktoken.get_encoding`` (the
  reference asks for the GPT-2 vocabulary in ``KG.__init__`` even when byte-pair encoding is off, which needs a
  download);
* a seeded synthetic KG of the configured shape written as ``train.txt`` (the same triples the other arm uses);
* a global hook that counts steps (``forward`` pre-hook on the DDP wrapper for the GPU trainer, optimiser-step
  pre-hook for the CPU trainer), brackets steps ``W .. W+K`` with CUDA events (or a host clock on CPU) and then
  stops the run by raising.
"""
from __future__ import annotations

import importlib.util
import os
import shutil
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


class _StopBench(Exception):
    pass


def reference_available():
    if not os.path.isdir(os.path.join(REF, "dicee")):
        return False, "baseline/_ref/dicee is missing (the offline pip install of the reference sources was not done on this machine)"
    return True, ""


def _load_synthetic():
    path = os.path.join(os.path.dirname(HERE), "dice_embeddings_b200", "data", "synthetic.py")
    spec = importlib.util.spec_from_file_location("_bench_synthetic", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def prepare_imports():
    for p in (os.path.join(HERE, "shims"), REF):
        if p not in sys.path:
            sys.path.insert(0, p)
    try:
        import tiktoken

        class _ByteEnc:
            n_vocab = 50257

            def encode(self, s):
                return list(str(s).encode("utf-8")) or [0]

            def encode_batch(self, xs):
                return [self.encode(x) for x in xs]

            def decode(self, t):
                return bytes(int(i) & 0xFF for i in t).decode("utf-8", errors="replace")

        tiktoken.get_encoding = lambda name: _ByteEnc()
    except ModuleNotFoundError:
        pass


CONFIGS = {
    1: dict(model="Keci", p=0, q=1, scoring_technique="KvsAll", trainer="torchCPUTrainer", embedding_dim=32,
            batch_size=1024, lr=0.1, optim="Adam", label_smoothing_rate=0.0, shape="umls"),
    2: dict(model="ComplEx", scoring_technique="KvsAll", trainer="torchDDP", embedding_dim=256, batch_size=4096,
            lr=0.1, optim="Adam", label_smoothing_rate=0.1, shape="fb15k237"),
}


def write_config_kg(config: int, path: str, seed: int = 0) -> str:
    syn = _load_synthetic()
    if CONFIGS[config]["shape"] == "umls":
        return syn.make_umls_like(path, seed)
    return syn.make_fb15k237_like(path, seed)


def run(config: int, gpus: int, steps: int, warmup: int, num_core: int = 0) -> dict:
    import torch
    prepare_imports()
    import dicee  # noqa: F401  (the reference)
    from dicee.config import Namespace
    from dicee.executer import Execute

    cfg = CONFIGS[config]
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if cfg["trainer"] == "torchDDP":
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        os.environ.setdefault("RANK", "0")
        os.environ.setdefault("LOCAL_RANK", "0")
        os.environ.setdefault("WORLD_SIZE", "1")
    base = os.environ.get("DICE_BENCH_TMP") or os.path.join(tempfile.gettempdir(), f"dice_ref_bench_c{config}")
    kg_dir, run_dir = os.path.join(base, "kg"), os.path.join(base, "run")
    if rank == 0:
        shutil.rmtree(base, ignore_errors=True)
        os.makedirs(base, exist_ok=True)
        write_config_kg(config, kg_dir)
        open(os.path.join(base, "ready"), "w").close()
    else:
        t0 = time.time()
        while not os.path.exists(os.path.join(base, "ready")) and time.time() - t0 < 600:
            time.sleep(0.2)

    args = Namespace()
    args.dataset_dir = kg_dir
    args.path_to_store_single_run = run_dir
    args.model = cfg["model"]
    args.scoring_technique = cfg["scoring_technique"]
    args.trainer = cfg["trainer"]
    args.embedding_dim = cfg["embedding_dim"]
    args.batch_size = cfg["batch_size"]
    args.lr = cfg["lr"]
    args.optim = cfg["optim"]
    args.label_smoothing_rate = cfg["label_smoothing_rate"]
    args.num_epochs = 10 ** 6          # the hook below ends the run after warmup + steps
    args.eval_model = "None"           # no evaluation; with this setting the reference adds no reciprocal triples
    args.num_core = int(num_core)      # the reference's own flag (DataLoader workers); 0 is its default
    args.random_seed = 0
    args.p, args.q = cfg.get("p", 0), cfg.get("q", 1)

    on_gpu = cfg["trainer"] == "torchDDP"
    top_level = "DistributedDataParallel" if on_gpu else cfg["model"]
    state = {"n": 0, "t0": None, "t1": None, "e0": None, "e1": None}

    def tick():
        n = state["n"]
        if n == warmup:
            if on_gpu:
                torch.cuda.synchronize()
                state["e0"] = torch.cuda.Event(enable_timing=True)
                state["e0"].record()
            state["t0"] = time.perf_counter()
        elif n == warmup + steps:
            if on_gpu:
                state["e1"] = torch.cuda.Event(enable_timing=True)
                state["e1"].record()
                torch.cuda.synchronize()
            state["t1"] = time.perf_counter()
            raise _StopBench()
        state["n"] = n + 1
        return None

    if on_gpu:
        # the DDP trainer calls ``ddp_model(source)`` once per step
        def hook(module, inputs):
            if type(module).__name__ == top_level and module.training:
                tick()
            return None
        handle = torch.nn.modules.module.register_module_forward_pre_hook(hook)
    else:
        # the CPU trainer calls ``model.training_step`` → ``self.forward`` directly (no module hooks fire), so
        # steps are counted at ``optimizer.step``
        from torch.optim.optimizer import register_optimizer_step_pre_hook
        handle = register_optimizer_step_pre_hook(lambda opt, a, k: tick())
    exe = Execute(args)
    try:
        exe.start()
        raise RuntimeError("reference finished before the requested number of steps")
    except _StopBench:
        pass
    finally:
        handle.remove()
    ms = state["e0"].elapsed_time(state["e1"]) if on_gpu else (state["t1"] - state["t0"]) * 1e3
    if on_gpu and world > 1 and torch.distributed.is_initialized():
        t = torch.tensor([ms], device="cuda")
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms = float(t.item())

    # number of training triples represented by one data point (unique (h, r) pair)
    import numpy as np
    train = np.load(os.path.join(run_dir, "train_set.npy")) if os.path.exists(os.path.join(run_dir, "train_set.npy")) \
        else np.asarray(exe.knowledge_graph.train_set)
    num_triples = int(train.shape[0])
    num_pairs = int(np.unique(train[:, 0].astype(np.int64) * (int(train[:, 1].max()) + 1) + train[:, 1]).shape[0])
    num_entities = int(max(train[:, 0].max(), train[:, 2].max())) + 1
    num_relations = int(train[:, 1].max()) + 1
    B = cfg["batch_size"]
    triples_per_step = B * world * num_triples / num_pairs
    if torch.distributed.is_initialized():
        try:
            torch.distributed.destroy_process_group()
        except Exception:
            pass
    return {"ms_total": ms, "steps": steps, "warmup": warmup, "world": world, "rank": rank,
            "triples_per_step": triples_per_step, "num_pairs": num_pairs, "num_triples": num_triples,
            "num_entities": num_entities, "num_relations": num_relations, "batch_size": B, "num_core": int(num_core),
            "h2d_bytes_per_step": B * 2 * 8 + B * num_entities * 4, "d2h_bytes_per_step": 4, "config": cfg}


def run_eval(gpus: int = 1) -> dict:
    """Filtered link-prediction evaluation of the reference on the config-2 graph shape (14 541 entities, 237
    relations, 272 115 train / 17 535 valid / 20 466 test triples): ``Execute(args).start()`` with one training epoch
    and ``eval_model='test'``; the wall-clock time of the reference's own ``Evaluator.eval`` call is measured by a
    wrapper around that method (the stock code runs it on the CPU after moving the model there)."""
    import numpy as np
    import torch  # noqa: F401
    prepare_imports()
    if not hasattr(np, "Inf"):
        # the reference's evaluator spells infinity ``np.Inf`` (dicee/evaluation/evaluator.py:461), an alias NumPy 2
        # dropped; the installed NumPy gets the alias back, the reference's files stay as they are
        np.Inf = np.inf
    import dicee  # noqa: F401
    from dicee.config import Namespace
    from dicee.evaluation import evaluator as ev_mod
    from dicee.executer import Execute
    syn = _load_synthetic()
    base = os.environ.get("DICE_BENCH_TMP") or os.path.join(tempfile.gettempdir(), "dice_ref_bench_eval")
    shutil.rmtree(base, ignore_errors=True)
    kg_dir, run_dir = os.path.join(base, "kg"), os.path.join(base, "run")
    syn.make_fb15k237_like(kg_dir, 0, with_eval_splits=True)
    args = Namespace()
    args.dataset_dir, args.path_to_store_single_run = kg_dir, run_dir
    args.model, args.scoring_technique, args.embedding_dim = "ComplEx", "KvsAll", 256
    args.batch_size, args.lr, args.optim, args.num_epochs = 4096, 0.1, "Adam", 1
    args.trainer = "torchCPUTrainer"
    args.eval_model, args.num_core, args.random_seed = "test", 0, 0
    timing = {}
    stock = ev_mod.Evaluator.eval

    def timed_eval(self, *a, **k):
        t0 = time.perf_counter()
        out = stock(self, *a, **k)
        timing["s"] = time.perf_counter() - t0
        return out

    ev_mod.Evaluator.eval = timed_eval
    try:
        report = Execute(args).start()
    finally:
        ev_mod.Evaluator.eval = stock
    test = np.load(os.path.join(run_dir, "test_set.npy"))
    return {"seconds": timing["s"], "queries": int(test.shape[0]), "num_entities": int(report["num_entities"]),
            "test_mrr": report.get("Test", {}).get("MRR"), "device": "cpu (the stock code moves the model there)"}
