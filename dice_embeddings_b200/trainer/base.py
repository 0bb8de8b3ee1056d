"""Trainer and callback base classes.

Hook names are the Lightning-style ones used throughout the reference (``on_fit_start``,
``on_train_epoch_start``, ``on_train_epoch_end``, ``on_train_batch_end``, ``on_fit_end``;
reference ``dicee/abstracts.py:18-150, 474-581``) so user callbacks written against it keep working.
"""
from __future__ import annotations

from typing import Iterator, List, Optional

import torch


class AbstractCallback:
    """Base class: every hook is a no-op."""

    def on_init_start(self, *args, **kwargs):
        pass

    def on_init_end(self, *args, **kwargs):
        pass

    def on_fit_start(self, trainer, model):
        pass

    def on_train_epoch_start(self, trainer, model):
        pass

    def on_train_epoch_end(self, trainer, model):
        pass

    def on_train_batch_end(self, *args, **kwargs):
        pass

    def on_fit_end(self, trainer, model):
        pass


class BatchLoader:
    """Iterable over device-resident batches of a :class:`BatchedDataset`.

    Stands where the reference puts a ``torch.utils.data.DataLoader`` (``dice_trainer.py:257-264``): it has
    ``dataset``, ``batch_size`` and ``__len__`` but builds each batch with tensor ops on the dataset's device
    instead of collating Python items in worker processes."""

    def __init__(self, dataset, batch_size: int, shuffle: bool = True, seed: int = 0, rank: int = 0,
                 world_size: int = 1, drop_last: bool = False, pad_last: bool = False, num_workers: int = 0):
        self.dataset = dataset
        self.batch_size = int(batch_size)
        self.shuffle = shuffle
        self.rank, self.world_size = rank, world_size
        self.drop_last = drop_last
        self.pad_last = pad_last          # full final batch by wrap-around (engines with a fixed batch size)
        self.num_workers = max(int(num_workers or 0), 0)   # ``--num_core``: batches are built ahead by a thread
        self.generator = torch.Generator()
        self.seed = int(seed)
        self.epoch = 0
        self.collate_fn = getattr(dataset, "collate_fn", None)

    def set_epoch(self, epoch: int) -> None:
        self.epoch = int(epoch)

    def __len__(self) -> int:
        return self.dataset.num_batches(self.batch_size, self.world_size, self.drop_last and not self.pad_last)

    def _batches(self) -> Iterator[tuple]:
        return self.dataset.batches(self.batch_size, self.shuffle, self.generator, self.rank, self.world_size,
                                    self.drop_last, self.pad_last)

    def __iter__(self) -> Iterator[tuple]:
        # same permutation on every rank: seed depends on (seed, epoch) only
        self.generator.manual_seed(self.seed * 1_000_003 + self.epoch)
        if self.num_workers > 0:
            yield from _prefetch(self._batches(), depth=2 * self.num_workers)
        else:
            yield from self._batches()
        self.epoch += 1


def _prefetch(it: Iterator[tuple], depth: int) -> Iterator[tuple]:
    """Run ``it`` in a background thread, ``depth`` batches ahead of the consumer (the role of the reference's
    DataLoader workers, ``dicee/trainer/dice_trainer.py:262-264``; batch construction here is tensor code that
    releases the interpreter lock, so a thread is enough).  Batches arrive in the same order as without it."""
    import queue
    import threading
    q: "queue.Queue" = queue.Queue(maxsize=max(depth, 1))
    end, stop = object(), threading.Event()

    def work():
        try:
            for item in it:
                while not stop.is_set():
                    try:
                        q.put(item, timeout=0.1)
                        break
                    except queue.Full:
                        continue
                if stop.is_set():
                    return
            q.put(end)
        except BaseException as exc:   # noqa: BLE001 - re-raised in the consumer
            q.put(exc)

    t = threading.Thread(target=work, daemon=True)
    t.start()
    try:
        while True:
            item = q.get()
            if item is end:
                return
            if isinstance(item, BaseException):
                raise item
            yield item
    finally:
        stop.set()


class AbstractTrainer:
    """Holds the argument namespace and dispatches callbacks."""

    def __init__(self, args, callbacks: Optional[List] = None):
        self.attributes = args
        self.callbacks = callbacks if callbacks is not None else []
        self.is_global_zero = True
        self.global_rank = 0
        self.local_rank = 0
        self.strategy = None
        self.current_epoch = 0
        self.model = None
        self.optimizer = None
        self.evaluator = None
        self.dataset = None
        self.form_of_labelling = None
        seed = getattr(args, "random_seed", 0) or 0
        torch.manual_seed(seed)
        if torch.cuda.is_available():
            torch.cuda.manual_seed_all(seed)

    @property
    def optimizers(self):
        return [self.optimizer]

    def on_fit_start(self, *args, **kwargs):
        for c in self.callbacks:
            c.on_fit_start(*args, **kwargs)

    def on_fit_end(self, *args, **kwargs):
        for c in self.callbacks:
            c.on_fit_end(*args, **kwargs)

    def on_train_epoch_start(self, *args, **kwargs):
        for c in self.callbacks:
            c.on_train_epoch_start(*args, **kwargs)

    def on_train_epoch_end(self, *args, **kwargs):
        for c in self.callbacks:
            c.on_train_epoch_end(*args, **kwargs)

    def on_train_batch_start(self, *args, **kwargs):
        for c in self.callbacks:
            hook = getattr(c, "on_train_batch_start", None)
            if hook is not None:
                hook(*args, **kwargs)

    def on_train_batch_end(self, *args, **kwargs):
        for c in self.callbacks:
            c.on_train_batch_end(*args, **kwargs)

    @staticmethod
    def save_checkpoint(full_path: str, model) -> None:
        torch.save(model.state_dict(), full_path)
