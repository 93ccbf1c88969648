"""``SRSgd`` (mirrors shared_ffi/optim_sr.py:7-114): SGD + weight decay + optional momentum with stochastic
rounding for bf16 parameters; fp32 parameters take plain SGD."""
import torch
from torch.optim import Optimizer

from .sr_triton import sgd_update


class SRSgd(Optimizer):
    def __init__(self, params, lr: float = 1e-3, weight_decay: float = 0.0, momentum: float = 0.0,
                 use_momentum: bool = True, stochastic_rounding: bool = True, seed: int = 123,
                 *, rng: str = "reference", contract: bool = True):
        defaults = dict(lr=lr, weight_decay=weight_decay, momentum=momentum, use_momentum=use_momentum,
                        stochastic_rounding=stochastic_rounding, seed=seed, rng=rng, contract=contract, step_count=0)
        super().__init__(params, defaults)

    # keys this class adds to a parameter group; a state dict written by the reference's SRSgd has none of them
    _EXTRA_GROUP_KEYS = dict(rng="reference", contract=True, step_count=0)

    def __setstate__(self, state):
        """``Optimizer.load_state_dict`` replaces the parameter groups with the saved ones.  Groups saved by the
        reference's optimizer (keys lr, weight_decay, momentum, use_momentum, stochastic_rounding, seed:
        shared_ffi/optim_sr.py:25-32) get the additive keys of this class back, at the values under which this class
        behaves like the reference."""
        super().__setstate__(state)
        for group in self.param_groups:
            for k, v in self._EXTRA_GROUP_KEYS.items():
                group.setdefault(k, v)

    def _momentum_buf(self, p, needed):
        # The reference allocates an fp32 buffer for every parameter even with momentum off
        # (optim_sr.py:36-44); here it is created on first use only.
        state = self.state[p]
        if needed and "momentum_buf" not in state:
            state["momentum_buf"] = torch.zeros_like(p.data, dtype=torch.float32)
        return state.get("momentum_buf")

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            lr, wd, mu = group["lr"], group["weight_decay"], group["momentum"]
            use_mom, sr, seed = group["use_momentum"], group["stochastic_rounding"], group["seed"]
            step = group["step_count"]
            group["seed"] += 1          # a new rounding pattern every step (optim_sr.py:59-62)
            group["step_count"] += 1
            mom_on = bool(use_mom and mu != 0.0)
            for p in group["params"]:
                if p.grad is None:
                    continue
                grad = p.grad
                if p.dtype == torch.float32:
                    if wd != 0.0:
                        grad = grad.add(p, alpha=wd)
                    if mom_on:
                        buf = self._momentum_buf(p, True)
                        buf.mul_(mu).add_(grad)
                        grad = buf
                    p.add_(grad, alpha=-lr)
                    continue
                w = p.data
                w_c = w if w.is_contiguous() else w.contiguous()
                g_c = grad if grad.is_contiguous() else grad.contiguous()
                # packed stream: 1-D parameters (bias) get their own key so they do not reuse column 0's bits
                pseed = seed ^ 0x62696173 if (group["rng"] == "packed" and p.dim() < 2) else seed
                sgd_update(w_c, g_c, self._momentum_buf(p, mom_on), learning_rate=lr, weight_decay=wd, momentum=mu,
                           use_momentum=use_mom, stochastic_rounding=sr, seed=pseed, rng=group["rng"], step=step,
                           contract=group["contract"])
                if w_c.data_ptr() != w.data_ptr():
                    p.data.copy_(w_c)
        return loss
