"""Checkpoints in the reference's de-facto layout, for every strategy.

The reference has no save/resume; what it fixes is the layout a checkpoint must
have to be interchangeable with it (tandem/zero.py:204-214,327-336;
tandem/optim.py:14-25): wrappers hold the model as `.module`, so parameter keys
are `module.<gpt key>`; ZeRO's flat order is `module.parameters()` order, FSDP's
is per unit in `units()` order; rank r's shard is chunk r of
torch.tensor_split(numel, world); optimizer state per key ("flat" for ZeRO-1/2,
the unit index for FSDP) is [step, exp_avg, exp_avg_sq] over that shard.

A checkpoint written here holds FULL tensors (gathered), so it can be loaded at
any world size and by any strategy:
    {"model": {"module.<name>": tensor}, "optim": {"kind", "hyper", "step", "exp_avg": {name: t}, "exp_avg_sq": {name: t}}, "extra": ...}
All functions are collective: every rank calls them; rank 0 writes the file.
"""

import torch

from .parallel.optim import ShardedAdamW
from .parallel.zero import FSDP, ZeRO, split_sizes


def _module(wrapped):
    return wrapped.module if hasattr(wrapped, "module") else wrapped


def _named(wrapped):
    return [("module." + n, p) for n, p in _module(wrapped).named_parameters()]


def _gather_flat(g, shard, numel, world):
    """All ranks' shards of a flat tensor, concatenated (on the shard's device)."""
    sizes = split_sizes(numel, world)
    full = torch.zeros(numel, dtype=shard.dtype, device=shard.device)
    lo = sum(sizes[:g.rank])
    full[lo:lo + sizes[g.rank]].copy_(shard)
    g.all_gather(full, sizes)
    return full


@torch.no_grad()
def full_state_dict(wrapped):
    """{"module.<name>": full CPU tensor} (gathers the shards of an FSDP wrapper)."""
    out = {}
    if isinstance(wrapped, FSDP):
        flat = wrapped.full_parameters().cpu()
        at = 0
        names = {id(p): n for n, p in _named(wrapped)}
        for u in wrapped.units:
            for p in u.flat.params:
                shape = wrapped._shapes[id(p)] if hasattr(wrapped, "_shapes") else p.shape
                n = u.flat.offset[p]
                size = _numel_of(u, p)
                out[names[id(p)]] = flat[at + n:at + n + size].view(shape).clone()
            at += u.flat.numel
        return out
    for name, p in _named(wrapped):
        out[name] = p.detach().cpu().clone()
    return out


def _numel_of(u, p):
    offs = sorted(u.flat.offset.values()) + [u.flat.numel]
    return offs[offs.index(u.flat.offset[p]) + 1] - u.flat.offset[p]


@torch.no_grad()
def load_full_state_dict(wrapped, sd):
    """Loads full tensors into any wrapper (an FSDP wrapper keeps only its shards)."""
    if isinstance(wrapped, FSDP):
        names = {id(p): n for n, p in _named(wrapped)}
        for u in wrapped.units:
            full = torch.empty(u.flat.numel, dtype=u.shard.dtype)
            for p in u.flat.params:
                a = u.flat.offset[p]
                t = sd[names[id(p)]].reshape(-1)
                full[a:a + t.numel()].copy_(t)
            u.shard.copy_(full[u.flat.lo:u.flat.hi])
        if wrapped.g.fused and wrapped.units[0].shard.is_cuda:
            wrapped.g._sym.device_barrier()
        return
    for name, p in _named(wrapped):
        p.copy_(sd[name])


@torch.no_grad()
def optimizer_state(wrapped, opt):
    """The optimizer's state as full per-parameter tensors."""
    g = getattr(wrapped, "g", None)
    if isinstance(opt, ShardedAdamW):
        hyper = {"lr": opt.lr, "betas": tuple(opt.betas), "eps": opt.eps, "weight_decay": opt.weight_decay}
        out = {"kind": "adamw", "hyper": hyper, "step": 0.0, "exp_avg": {}, "exp_avg_sq": {}, "master": {}}
        names = {id(p): n for n, p in _named(wrapped)}
        layouts = [("flat", wrapped.flat)] if isinstance(wrapped, ZeRO) else [(u.index, u.flat) for u in wrapped.units]
        for key, layout in layouts:
            if key not in opt.state:
                continue
            step, m, v = opt.state[key]
            # with step constants kept on the device (graph replay) the host-side count only saw the recorded step
            out["step"] = opt.steps_on_device() if opt.device_scalars() is not None else step
            parts = {"exp_avg": _gather_flat(g, m, layout.numel, g.size).cpu(),
                     "exp_avg_sq": _gather_flat(g, v, layout.numel, g.size).cpu()}
            if key in opt.master:  # 16-bit parameters: the fp32 master weights are optimizer state too
                parts["master"] = _gather_flat(g, opt.master[key], layout.numel, g.size).cpu()
            offs = sorted(layout.offset.values()) + [layout.numel]
            for p in layout.params:
                a = layout.offset[p]
                b = offs[offs.index(a) + 1]
                for kind, flat in parts.items():
                    out[kind][names[id(p)]] = flat[a:b].clone()
        return out
    if hasattr(opt, "slots") and opt.slots and "sizes" in opt.slots[0]:  # ShardedBucketAdamW: each rank holds chunk r of every span
        names = {id(p): n for n, p in _named(wrapped)}
        out = {"kind": "adamw", "hyper": {"lr": opt.rule.lr, "betas": tuple(opt.rule.betas), "eps": opt.rule.eps,
                                          "weight_decay": opt.rule.weight_decay},
               "step": opt.step_count, "exp_avg": {}, "exp_avg_sq": {}, "master": {}}
        for s in opt.slots:
            span = s["bucket"]
            parts = {}
            for kind, key in (("exp_avg", "m"), ("exp_avg_sq", "v"), ("master", "master")):
                full = torch.zeros(span.hi - span.lo, dtype=s[key].dtype, device=s[key].device)
                full[s["lo"]:s["lo"] + s[key].numel()].copy_(s[key])
                g.all_gather(full, s["sizes"])
                parts[kind] = full.cpu()
            at = 0
            for p in span.params:
                n = p.numel()
                for kind, full in parts.items():
                    out[kind][names[id(p)]] = full[at:at + n].clone()
                at += n
        return out
    if hasattr(opt, "slots"):  # BucketAdamW: replicated state, bucket-major
        names = {id(p): n for n, p in _named(wrapped)}
        out = {"kind": "adamw", "hyper": {"lr": opt.rule.lr, "betas": tuple(opt.rule.betas), "eps": opt.rule.eps,
                                          "weight_decay": opt.rule.weight_decay},
               "step": opt.step_count, "exp_avg": {}, "exp_avg_sq": {}, "master": {}}
        for s in opt.slots:
            at = 0
            for p in s["bucket"].params:
                n = p.numel()
                out["exp_avg"][names[id(p)]] = s["m"][at:at + n].detach().cpu().clone()
                out["exp_avg_sq"][names[id(p)]] = s["v"][at:at + n].detach().cpu().clone()
                out["master"][names[id(p)]] = s["master"][at:at + n].detach().cpu().clone()
                at += n
        return out
    return {"kind": "torch", "state": opt.state_dict()}


@torch.no_grad()
def load_optimizer_state(wrapped, opt, state):
    if state["kind"] == "torch":
        opt.load_state_dict(state["state"])
        return
    names = {id(p): n for n, p in _named(wrapped)}
    if isinstance(opt, ShardedAdamW):
        h = state["hyper"]
        opt.lr, opt.betas, opt.eps, opt.weight_decay = h["lr"], tuple(h["betas"]), h["eps"], h["weight_decay"]
        layouts = [("flat", wrapped.flat, wrapped.buf)] if isinstance(wrapped, ZeRO) else [(u.index, u.flat, u.shard) for u in wrapped.units]
        saved_master = state.get("master") or {}
        for key, layout, like in layouts:
            shard = like[layout.lo:layout.hi] if like.numel() == layout.numel else like  # ZeRO passes the whole buffer
            sixteen = like.dtype in (torch.bfloat16, torch.float16)
            wide = torch.float64 if like.dtype == torch.float64 else torch.float32
            fm = torch.zeros(layout.numel, dtype=wide)
            fv = torch.zeros(layout.numel, dtype=wide)
            fw = torch.zeros(layout.numel, dtype=wide) if sixteen else None
            have_master = sixteen
            for p in layout.params:
                a = layout.offset[p]
                name = names[id(p)]
                m, v = state["exp_avg"][name], state["exp_avg_sq"][name]
                fm[a:a + m.numel()].copy_(m.reshape(-1))
                fv[a:a + v.numel()].copy_(v.reshape(-1))
                if sixteen:
                    if name in saved_master:
                        fw[a:a + m.numel()].copy_(saved_master[name].reshape(-1))
                    else:
                        have_master = False
            dev = like.device
            # Moments (and the master copy) of a 16-bit shard stay fp32: the update kernels address them as float.
            opt.state[key] = [float(state["step"]), fm[layout.lo:layout.hi].to(dev).clone(), fv[layout.lo:layout.hi].to(dev).clone()]
            if sixteen:
                # a checkpoint written from fp32 training has no master: start it from the (just loaded) parameters
                opt.master[key] = fw[layout.lo:layout.hi].to(dev).clone() if have_master else shard.detach().to(wide).clone()
            else:
                opt.master.pop(key, None)
        if opt.device_scalars() is not None:
            opt._step_dev.fill_(float(state["step"]))
            opt.advance_on_device()  # the constants of the step that comes next
        return
    opt.step_count = float(state["step"])
    sharded = bool(opt.slots) and "sizes" in opt.slots[0]
    if hasattr(opt, "_step_dev"):
        opt._step_dev.fill_(opt.step_count)
        if sharded:
            opt._prepare()  # the sharded optimizer keeps the NEXT step's constants ready on the device
        elif getattr(opt, "during_backward", False):
            opt._prepare_next()  # so does the replicated one when it updates during backward
    for s in opt.slots:
        span = s["bucket"]
        if sharded:
            full = {k: torch.zeros(span.hi - span.lo, dtype=s["m"].dtype) for k in ("m", "v", "master")}
        at = 0
        for p in span.params:
            n = p.numel()
            name = names[id(p)]
            if sharded:
                full["m"][at:at + n].copy_(state["exp_avg"][name].reshape(-1))
                full["v"][at:at + n].copy_(state["exp_avg_sq"][name].reshape(-1))
                source = state["master"][name] if name in (state.get("master") or {}) else p.detach().cpu().to(s["m"].dtype)
                full["master"][at:at + n].copy_(source.reshape(-1))
            else:
                s["m"][at:at + n].copy_(state["exp_avg"][name])
                s["v"][at:at + n].copy_(state["exp_avg_sq"][name])
                if s["master"] is not s["flat"] and "master" in state:
                    s["master"][at:at + n].copy_(state["master"][name])
            at += n
        if sharded:
            lo, count = s["lo"], s["m"].numel()
            s["m"].copy_(full["m"][lo:lo + count])
            s["v"].copy_(full["v"][lo:lo + count])
            if s["master"].data_ptr() != s["flat"][lo:lo + count].data_ptr():
                s["master"].copy_(full["master"][lo:lo + count])


def save(path, wrapped, opt=None, extra=None):
    """Collective.  Rank 0 writes {"model", "optim", "extra"} to `path`."""
    g = getattr(wrapped, "g", None)
    blob = {"model": full_state_dict(wrapped), "optim": optimizer_state(wrapped, opt) if opt is not None else None, "extra": extra}
    if g is None or g.rank == 0:
        torch.save(blob, path)
    if g is not None:
        g.barrier()


def load(path, wrapped, opt=None):
    """Collective.  Every rank reads `path`; returns the saved `extra`."""
    blob = torch.load(path, weights_only=False, map_location="cpu")
    load_full_state_dict(wrapped, blob["model"])
    if opt is not None and blob["optim"] is not None:
        load_optimizer_state(wrapped, opt, blob["optim"])
    return blob["extra"]
