"""``GroupFixedFanIn`` (mirrors shared_ffi/rewire.py:36-239): the grouped fixed-fan-in sparse linear layer
with prune/regrow rewiring; the tensor math of ``rewire`` runs in one CUDA kernel."""
import math

import torch

from . import ops
from .. import ffi as _ffi

GROWTH_MODES = ['random']
PRUNE_MODES = ['threshold', 'fraction']
INIT_MODES = ["random", "zero"]
REGROW_MODES = ["replace", "unused"]


class GroupFixedFanIn(torch.nn.Module):
    """Each of ``out_features`` labels reads ``fan_in`` inputs; ``group_size`` consecutive labels share one
    index row of the ``group_locations`` buffer [num_groups, fan_in] (int32).

    Constructor arguments are the reference's.  Keyword-only additions: ``regrow`` ('replace' = uniform with
    replacement as in the reference; 'unused' = only indices the row does not hold yet), ``regroup`` (sort
    every index row after rewiring and permute the weight columns with it) and ``seed`` for the Philox draws.
    """
    __constants__ = ['in_features', 'out_features', 'fan_in']

    def __init__(self, in_features: int, out_features: int, fan_in: int, bias: bool = True, device=None, dtype=None, *,
                 group_size=32, prune_mode="threshold", rewire_threshold=None, rewire_fraction=None, growth_mode="random",
                 init_mode="random", regrow="replace", regroup=False, seed=0, **kwargs):
        super().__init__(**kwargs)
        factory_kwargs = {'device': device, 'dtype': dtype}
        self.in_features, self.out_features, self.fan_in = in_features, out_features, fan_in
        assert prune_mode in PRUNE_MODES, f"Invalid prune_mode={prune_mode}; supported: {PRUNE_MODES}"
        assert growth_mode in GROWTH_MODES, f"Invalid growth_mode={growth_mode}; supported: {GROWTH_MODES}"
        assert init_mode in INIT_MODES, f"Invalid init_mode={init_mode}; supported: {INIT_MODES}"
        assert regrow in REGROW_MODES, f"Invalid regrow={regrow}; supported: {REGROW_MODES}"
        if prune_mode == "threshold" and rewire_threshold is None:
            raise ValueError("rewire_threshold must be specified for prune_mode 'threshold'")
        elif prune_mode == "fraction" and rewire_fraction is None:
            raise ValueError("rewire_fraction must be specified for prune_mode 'fraction'")
        self.prune_mode, self.growth_mode, self.init_mode = prune_mode, growth_mode, init_mode
        self.regrow, self.regroup, self.seed = regrow, bool(regroup), int(seed)
        self._rewire_calls = 0
        if prune_mode == 'fraction':
            self.rewire_fraction = rewire_fraction
            assert 0 <= rewire_fraction < 1, f"Invalid reware_fraction={rewire_fraction}; supported range [0,1)"
        else:
            self.rewire_threshold = rewire_threshold

        weights = torch.empty((out_features, fan_in), **factory_kwargs)
        self.weights = torch.nn.parameter.Parameter(weights)
        bound = 1 / math.sqrt(self.fan_in)
        torch.nn.init.uniform_(self.weights, -bound, bound)
        if bias:
            self.bias = torch.nn.parameter.Parameter(torch.empty(out_features, **factory_kwargs))
            torch.nn.init.zeros_(self.bias)
        else:
            self.register_parameter('bias', None)
        assert group_size in [16, 32, 64, 128], f"Supported group sizes: 16, 32, 64, 128. Selected group size={group_size}"
        assert fan_in % 16 == 0 and 16 <= fan_in <= 128, f"fan_in must be a multiple of 16 in [16,128], got {fan_in}"
        self.group_size = group_size
        self.num_groups = (out_features + self.group_size - 1) // self.group_size
        group_locations = torch.randint(high=self.in_features, size=(self.num_groups, fan_in), dtype=torch.int32)
        self.register_buffer("group_locations", group_locations.to(self.weights.device), persistent=True)

    def forward(self, features):
        return ops.group_ffi_mul(features, self.weights, self.group_locations, self.bias, gsize=self.group_size)

    def extra_repr(self) -> str:
        return 'in_features={}, out_features={}, fan_in={}, bias={}'.format(
            self.in_features, self.out_features, self.fan_in, self.bias is not None)

    @torch.no_grad()
    def rewire(self, momentum_buf=None):
        """Group-wise prune + regrow (rewire.py:143-239).  For each group: score_j = mean over rows of |w|;
        prune low-score slots; draw new input indices for them (shared by all rows of the group);
        re-initialise those weight columns ('zero' or U(+-1/sqrt(fan_in))).  ``momentum_buf`` (fp32, same shape
        as ``weights``) is kept consistent when given.  Returns the number of pruned (group, slot) pairs."""
        if self.out_features == 0:
            return 0
        if self.prune_mode == 'fraction':
            n_prune = int(self.fan_in * self.rewire_fraction)
            if n_prune == 0:
                return 0
            mode, thr = 1, 0.0
        else:
            n_prune, mode, thr = 0, 0, float(self.rewire_threshold)
        changed = torch.zeros(1, dtype=torch.int32, device=self.weights.device)
        _ffi.rewire(self.weights.data, self.group_locations, momentum_buf, self.in_features, self.group_size, 0, mode, thr,
                    n_prune, {'replace': 0, 'unused': 1}[self.regrow], {'zero': 0, 'random': 1}[self.init_mode], self.regroup, self.seed,
                    self._rewire_calls, changed)
        self._rewire_calls += 1
        return int(changed.item())
