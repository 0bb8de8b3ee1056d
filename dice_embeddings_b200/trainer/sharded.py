"""``--trainer Sharded``: the row-sharded fused engines as a trainer of their own.

KvsAll / AllvsAll / 1vsAll use :class:`~dice_embeddings_b200.parallel.sharded_engine.ShardedKvsAllEngine` (the same
engine that ``torchDDP`` selects when the model is covered, but here it is mandatory); NegSample / 1vsSample /
KvsSample use :class:`~dice_embeddings_b200.parallel.sharded_sampled.ShardedSampledEngine`, whose row-wise sparse
optimiser decays the moments of a row only when the row receives a gradient.  ``torchDDP`` keeps the dense update of
the reference for those techniques, which is why the sampled engine is reached through this trainer only."""
from __future__ import annotations

from .ddp import TorchDDPTrainer


class ShardedTrainer(TorchDDPTrainer):
    def _maybe_sharded_engine(self, model, loader):
        st = getattr(self.attributes, "scoring_technique", None)
        from ..ops.sampled_step import SUPPORTED_SCORING as SAMPLED
        if self.world_size == 1:
            if st in SAMPLED:
                from ..ops.sampled_step import build_sampled_engine
                return build_sampled_engine(model, loader.dataset, self.attributes, self.device, strict=True)
            from ..ops.fused_step import build_fused_engine
            return build_fused_engine(model, loader.dataset, self.attributes, self.device, strict=True)
        if st in SAMPLED:
            from ..ops import kernels as K
            from ..ops.sampled_step import sampled_model_code
            from ..parallel.sharded_sampled import ShardedSampledEngine
            if sampled_model_code(model) is None or K.OPT_CODE.get(model.optimizer_name, 9) > 2:
                raise RuntimeError("--trainer Sharded with a sampled scoring technique needs DistMult, ComplEx, QMult, "
                                   "OMult, Keci (p=0, q=1) or TransE and Adam / AdamW / SGD")
            ds = loader.dataset
            if st == "NegSample" and hasattr(ds, "defer_sampling"):
                ds.defer_sampling = True   # the engine draws the corruptions on the device
            a = self.attributes
            return ShardedSampledEngine(model, st, batch_size=loader.batch_size, lr=a.lr, neg_ratio=getattr(a, "neg_ratio", 0) or 0,
                                        label_smoothing=getattr(a, "label_smoothing_rate", 0.0) or 0.0,
                                        weight_decay=getattr(a, "weight_decay", 0.0) or 0.0, device=self.device,
                                        seed=getattr(a, "random_seed", 0) or 0)
        eng = super()._maybe_sharded_engine(model, loader)
        if eng is None:
            raise RuntimeError("--trainer Sharded needs B200 GPUs, a covered model (DistMult, ComplEx, QMult, OMult, "
                               "Keci p=0 q=1; dim 64/128/256) and KvsAll / AllvsAll / 1vsAll")
        return eng
