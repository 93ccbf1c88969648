"""Checkpoint interop between the reference's state dicts and the label-sharded layout.

The reference saves ``model.state_dict()`` (src/runner.py:304-321): for an FFI layer the entries
``<prefix>weights`` bf16 [L,F], ``<prefix>bias`` bf16 [L] and the persistent buffer ``<prefix>group_locations``
int32 [NG,F].  A second-stage model with one index row per label gets its ``locations`` [L,F] by repeating every
group row ``group_size`` times (src/runner.py:324-334, 352-389).  The reference does not save the optimizer's
rounding seed or momentum for the sharded case; here a shard's state carries them (``steps``, ``seed``,
``momentum``), so a resumed run draws the same random bits as an uninterrupted one.

Nothing here touches the GPU kernels: these are slices, concatenations and copies.
"""
import torch

from .fused import FusedFFIShard, shard_labels, split_groups_by_cost


def inflate_group_locations(group_locations, out_features, group_size):
    """[NG,F] -> [L,F]: every group row repeated ``group_size`` times, truncated to ``out_features`` rows
    (src/runner.py:324-334)."""
    return group_locations.repeat_interleave(int(group_size), dim=0)[:int(out_features)]


def find_key_end(state_dict, suffix):
    """First key ending in ``suffix`` (the reference looks entries up this way, src/runner.py:360-364)."""
    for k in state_dict.keys():
        if k.endswith(suffix):
            return k
    return None


def layer_tensors(state_dict, prefix):
    """(group_locations, weights, bias-or-None) of the FFI layer stored under ``prefix`` (e.g. 'tail_layer.').

    The three entries must belong to the same module: the module path is taken from the ``group_locations`` key
    (only FFI layers have that buffer), and ``weights`` / ``bias`` are looked up under exactly that path — a suffix
    search for 'bias' alone could pick an encoder's bias.  With an empty ``prefix`` the state dict must hold exactly
    one FFI layer."""
    cands = [k for k in state_dict.keys() if k == prefix + "group_locations" or (k.endswith("." + prefix + "group_locations") if prefix else k.endswith("group_locations"))]
    if len(cands) != 1:
        raise KeyError(f"expected exactly one '{prefix}group_locations' entry in the state dict, found {len(cands)}: {cands[:4]}")
    gk = cands[0]
    base = gk[:-len("group_locations")]
    wk, bk = base + "weights", base + "bias"
    if wk not in state_dict:
        raise KeyError(f"{wk} not found in the state dict")
    return state_dict[gk], state_dict[wk], state_dict.get(bk)


def shard_bounds(L, group_size, world_size, group_cost=None):
    """Group boundaries of every rank: ``world_size + 1`` non-decreasing values (count split or cost split)."""
    NG = (L + group_size - 1) // group_size
    if group_cost is not None:
        return split_groups_by_cost(group_cost, world_size)
    return [shard_labels(L, group_size, world_size, r)[2] for r in range(world_size)] + [NG]


def shard_state(shard, g0=None):
    """State of one ``FusedFFIShard``: its slice of the reference's three tensors (on the CPU), where the slice
    sits (first label, first group) and the update's random-stream position."""
    st = {"weights": shard.w.detach().cpu().clone(), "bias": None if shard.bias is None else shard.bias.detach().cpu().clone(),
          "group_locations": shard.loc.detach().cpu().clone(), "label0": int(shard.label0),
          "group0": int(shard.label0 // shard.G if g0 is None else g0), "group_size": int(shard.G), "in_features": int(shard.D),
          "steps": int(shard.steps), "seed": int(shard.seed), "rng": shard.rng,
          "momentum_w": None if shard.mom_w is None else shard.mom_w.detach().cpu().clone(),
          "momentum_b": None if shard.mom_b is None else shard.mom_b.detach().cpu().clone()}
    return st


def load_shard_state(shard, st):
    """Inverse of ``shard_state`` for a shard that covers the same label range."""
    if int(st["label0"]) != int(shard.label0) or tuple(st["weights"].shape) != tuple(shard.w.shape):
        raise ValueError("the saved shard covers a different label range; merge the shards and re-split instead")
    shard.w.copy_(st["weights"].to(shard.w.device))
    if shard.bias is not None and st["bias"] is not None:
        shard.bias.copy_(st["bias"].to(shard.bias.device))
    shard.loc.copy_(st["group_locations"].to(shard.loc.device))
    shard.steps, shard.seed = int(st["steps"]), int(st["seed"])
    if shard.mom_w is not None and st.get("momentum_w") is not None:
        shard.mom_w.copy_(st["momentum_w"].to(shard.mom_w.device))
    if shard.mom_b is not None and st.get("momentum_b") is not None:
        shard.mom_b.copy_(st["momentum_b"].to(shard.mom_b.device))


def merge_shard_states(states, prefix=""):
    """Shard states of all ranks (any order) -> the reference's three state-dict entries for the whole layer."""
    states = sorted(states, key=lambda s: s["label0"])
    pos = 0
    for s in states:
        if int(s["label0"]) != pos:
            raise ValueError(f"shards do not tile the label range: expected a shard starting at label {pos}, got {s['label0']}")
        pos += s["weights"].shape[0]
    out = {prefix + "weights": torch.cat([s["weights"] for s in states]),
           prefix + "group_locations": torch.cat([s["group_locations"] for s in states])}
    if all(s["bias"] is not None for s in states):
        out[prefix + "bias"] = torch.cat([s["bias"] for s in states])
    return out


def split_layer(group_locations, weights, bias, group_size, bounds):
    """Whole-layer tensors -> per-rank (group_locations, weights, bias, label0) for the group ``bounds``."""
    L = weights.shape[0]
    parts = []
    for g0, g1 in zip(bounds, bounds[1:]):
        l0, l1 = min(L, g0 * group_size), min(L, g1 * group_size)
        parts.append((group_locations[g0:g1].contiguous(), weights[l0:l1].contiguous(), None if bias is None else bias[l0:l1].contiguous(), l0))
    return parts


def shard_from_state_dict(state_dict, prefix, group_size, in_features, rank, world_size, device, group_cost=None, **shard_kwargs):
    """Build this rank's ``FusedFFIShard`` from a reference checkpoint's state dict."""
    loc, w, b = layer_tensors(state_dict, prefix)
    bounds = shard_bounds(w.shape[0], group_size, world_size, group_cost)
    l, ww, bb, l0 = split_layer(loc, w, b, group_size, bounds)[rank]
    return FusedFFIShard(l.to(device), ww.to(device), None if bb is None else bb.to(device), group_size, in_features, label0=l0, **shard_kwargs)
