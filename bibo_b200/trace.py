"""Router mechanics during training, accumulated by the router and plan kernels themselves.

Host-side counterpart of the reference's ``RouterTrace`` (ablate/common/router_trace.py:67-168): the
same constructor arguments, the same ``flush()`` keys and ``close()``.  The reference hangs a
forward-pre-hook on every expert module and a forward hook on every router; each hook runs about
twenty small launches per layer (bincount, max / min / sum, an entropy, a second top-k for the boundary
gap).  Here the router kernel writes those per-token quantities as per-block sums and the plan kernel
folds them into this object's device buffers (``bibo_moe_router_trace`` in include/bibo_moe.h), so a
traced training forward launches exactly the kernels an untraced one does.  ``flush()`` makes the one
device-to-host transfer of an interval, as the reference's does.

Layers served: this package's ``BiBoMoELayer``, any layer of the reference's class whose forward was
replaced by ``bibo_b200.install`` (``moe.layer_forward`` reads ``layer._router_trace``) and the
expert-parallel ``ExpertParallelMoELayer`` (every rank traces its own tokens, as the reference's hooks
would).
"""
import math

import torch

# word order of the accumulator, fixed by the kernels (include/bibo_moe.h)
SPLIT_TOP1, ENTROPY, TOKENS, W_TOP1, W_SUM, W_MIN, GAP, FORWARDS = range(8)


class RouterTrace:
    def __init__(self, model, num_experts, device):
        self.E = int(num_experts)
        self.counts = torch.zeros(self.E, dtype=torch.float32, device=device)
        self.acc = torch.zeros(8, dtype=torch.float32, device=device)
        self._layers = [m for m in model.modules()
                        if m.__class__.__name__ in ("BiBoMoELayer", "ExpertParallelMoELayer") and hasattr(m, "gate")]
        first = getattr(self._layers[0], "experts", None) if self._layers else None
        # boundaries of the +Identity / -Identity experts, for the two special-load channels
        self.n_glu = int(getattr(first, "num_glu_experts", self.E))
        self.pos_end = int(getattr(first, "pos_end", self.E))
        for m in self._layers:
            m._router_trace = self

    def buffers(self, layer):
        """(acc, counts, gap) for ``functional.moe_forward(trace=...)``, or None for an eval forward: the
        reference's hooks skip those too (router_trace.py:108,115)."""
        return (self.acc, self.counts, None) if layer.training else None

    @torch.no_grad()
    def flush(self):
        """Metrics of the interval since the last flush, then reset.  One device->host transfer."""
        if self.E < 2:
            return {}
        a = self.acc
        tokens = a[TOKENS].clamp_min(1.0)
        load = self.counts / self.counts.sum().clamp_min(1.0)
        channels = {
            "train/balance_entropy": -(load * load.clamp_min(1e-12).log()).sum() / math.log(self.E),
            "train/router_top1_weight": a[SPLIT_TOP1] / tokens,
            "train/router_entropy": a[ENTROPY] / tokens,
            "train/max_expert_load": load.max(),
            "train/router_w_top1": a[W_TOP1] / tokens,
            "train/router_w_sum": a[W_SUM] / tokens,
            "train/router_w_min": a[W_MIN] / tokens,
            "train/special_load": load[self.n_glu:].sum(),
            "train/neg_identity_load": load[self.pos_end:].sum(),
            "train/router_boundary_gap": a[GAP] / a[FORWARDS].clamp_min(1.0),
        }
        values = torch.stack(list(channels.values()) + [a[TOKENS]]).cpu().tolist()
        self.counts.zero_()
        self.acc.zero_()
        if values[-1] < 1:
            return {}
        return dict(zip(channels.keys(), values[:-1]))

    def close(self):
        for m in self._layers:
            if getattr(m, "_router_trace", None) is self:
                m._router_trace = None
        self._layers = []
