"""``--trainer Sharded``: the row-sharded fused engine as a trainer of its own (same engine that ``torchDDP``
selects when the model is covered, but here it is mandatory)."""
from __future__ import annotations

from .ddp import TorchDDPTrainer


class ShardedTrainer(TorchDDPTrainer):
    def _maybe_sharded_engine(self, model, loader):
        if self.world_size == 1:
            from ..ops.fused_step import build_fused_engine
            return build_fused_engine(model, loader.dataset, self.attributes, self.device, strict=True)
        eng = super()._maybe_sharded_engine(model, loader)
        if eng is None:
            raise RuntimeError("--trainer Sharded needs B200 GPUs, a covered model (DistMult, ComplEx, QMult, OMult, "
                               "Keci p=0 q=1; dim 64/128/256) and KvsAll / AllvsAll / 1vsAll")
        return eng
