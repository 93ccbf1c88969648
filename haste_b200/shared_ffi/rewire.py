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
SCORE_MODES = ["mean", "max"]
PRUNE_SCOPES = ["group", "global"]


class GroupFixedFanIn(torch.nn.Module):
    """Each of ``out_features`` labels reads ``fan_in`` inputs; ``group_size`` consecutive labels share one
    index row of the ``group_locations`` buffer [num_groups, fan_in] (int32).

    Constructor arguments are the reference's.  Keyword-only additions: ``regrow`` ('replace' = uniform with
    replacement as in the reference; 'unused' = only indices the row does not hold yet), ``regroup`` (sort
    every index row after rewiring and permute the weight columns with it), ``seed`` for the Philox draws (None,
    the default, derives one from the layer's shape, so that two different layers do not draw the same indices),
    ``score_mode`` ('mean' or 'max' of |w| over a group's rows) and ``prune_scope`` ('group': the fraction is
    taken inside every group, as shared_ffi/rewire.py does; 'global': over all (group, slot) pairs of the layer,
    as src/group_fanin_real.py:232-250 does).
    """
    __constants__ = ['in_features', 'out_features', 'fan_in']

    def __init__(self, in_features: int, out_features: int, fan_in: int, bias: bool = True, device=None, dtype=None, *,
                 group_size=32, prune_mode="threshold", rewire_threshold=None, rewire_fraction=None, growth_mode="random",
                 init_mode="random", regrow="replace", regroup=False, seed=None, score_mode="mean", prune_scope="group", **kwargs):
        super().__init__(**kwargs)
        factory_kwargs = {'device': device, 'dtype': dtype}
        self.in_features, self.out_features, self.fan_in = in_features, out_features, fan_in
        assert prune_mode in PRUNE_MODES, f"Invalid prune_mode={prune_mode}; supported: {PRUNE_MODES}"
        assert growth_mode in GROWTH_MODES, f"Invalid growth_mode={growth_mode}; supported: {GROWTH_MODES}"
        assert init_mode in INIT_MODES, f"Invalid init_mode={init_mode}; supported: {INIT_MODES}"
        assert regrow in REGROW_MODES, f"Invalid regrow={regrow}; supported: {REGROW_MODES}"
        assert score_mode in SCORE_MODES, f"Invalid score_mode={score_mode}; supported: {SCORE_MODES}"
        assert prune_scope in PRUNE_SCOPES, f"Invalid prune_scope={prune_scope}; supported: {PRUNE_SCOPES}"
        if prune_mode == "threshold" and rewire_threshold is None:
            raise ValueError("rewire_threshold must be specified for prune_mode 'threshold'")
        elif prune_mode == "fraction" and rewire_fraction is None:
            raise ValueError("rewire_fraction must be specified for prune_mode 'fraction'")
        self.prune_mode, self.growth_mode, self.init_mode = prune_mode, growth_mode, init_mode
        if seed is None:
            seed = (in_features * 1000003 + out_features * 10007 + fan_in * 101 + group_size) & 0x7FFFFFFF
        self.regrow, self.regroup, self.seed = regrow, bool(regroup), int(seed)
        self.score_mode, self.prune_scope = score_mode, prune_scope
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

    # The position in the rewiring random stream (seed, number of rewire calls so far) travels with the state dict,
    # so that a resumed run continues the stream instead of replaying the draws of the first rewire.  State dicts
    # written by the reference have no such entry; loading them keeps the constructor's values.
    def get_extra_state(self):
        return {"rewire_seed": int(self.seed), "rewire_calls": int(self._rewire_calls)}

    def set_extra_state(self, state):
        if state:
            self.seed = int(state.get("rewire_seed", self.seed))
            self._rewire_calls = int(state.get("rewire_calls", self._rewire_calls))

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs)
        extra = prefix + "_extra_state"
        if extra in missing_keys:          # a reference checkpoint: nothing to restore, not an error
            missing_keys.remove(extra)

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
            if self.prune_scope == 'global':
                n_prune, mode = int(self.num_groups * self.fan_in * self.rewire_fraction), 2
            else:
                n_prune, mode = int(self.fan_in * self.rewire_fraction), 1
            if n_prune == 0:
                return 0
            thr = 0.0
        else:
            n_prune, mode, thr = 0, 0, float(self.rewire_threshold)
        changed = torch.zeros(1, dtype=torch.int32, device=self.weights.device)
        _ffi.rewire_ex(self.weights.data, self.group_locations, momentum_buf, self.in_features, self.group_size, 0,
                       SCORE_MODES.index(self.score_mode), mode, thr, n_prune, {'replace': 0, 'unused': 1}[self.regrow],
                       {'zero': 0, 'random': 1}[self.init_mode], self.regroup, self.seed, self._rewire_calls, changed)
        self._rewire_calls += 1
        return int(changed.item())


class GroupFixedFanInReal(GroupFixedFanIn):
    """The layer class the reference's model builds (src/group_fanin_real.py:34-286, src/model.py:188-204): same
    parameters and forward as ``GroupFixedFanIn``; ``rewire`` scores slots by the 'mean' or 'max' of |w| and, in
    'fraction' mode, prunes the lowest ``int(num_groups * fan_in * rewire_fraction)`` slots of the whole layer."""

    def __init__(self, in_features: int, out_features: int, fan_in: int, bias: bool = True, device=None, dtype=None, *,
                 group_size=32, prune_mode="threshold", rewire_threshold=None, rewire_fraction=None, growth_mode="random",
                 init_mode="random", score_mode="mean", **kwargs):
        super().__init__(in_features, out_features, fan_in, bias, device, dtype, group_size=group_size, prune_mode=prune_mode,
                         rewire_threshold=rewire_threshold, rewire_fraction=rewire_fraction, growth_mode=growth_mode,
                         init_mode=init_mode, score_mode=score_mode, prune_scope="global", **kwargs)
        self.use_grad = False
