"""AdamW over flat shards, for the ZeRO stages.

Arithmetic: torch.optim.AdamW's single-tensor path (foreach=False, not
capturable), operation for operation, as the reference's tandem/optim.py:11-40
does; every operation is elementwise, so a rank updating its shard of a flat
buffer produces the bits torch produces for those elements.  On a GPU the same
sequence runs as ONE fused kernel (tandem_b200/cuda/adamw.cu) that reads the
gradient, both moments and the parameter once and writes them once (optionally
also a bf16 copy of the parameter for the next forward); it evaluates the same
roundings in the same order.

state[key] = [step (float), exp_avg, exp_avg_sq]; key is "flat" for ZeRO-1/2 and
the unit index for FSDP.

Mixed precision: a 16-bit shard is never updated in its own precision.  The
optimizer keeps an fp32 master copy of the shard (master[key]) and fp32 moments,
steps those, and writes the shard back as the rounded copy of the master, in the
same kernel on a GPU.  (The reference trains in fp32 only.)
"""

import torch


class ShardedAdamW:
    def __init__(self, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2, fused=None):
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.fused = fused  # None: fused kernel on CUDA shards, torch ops elsewhere
        self.state = {}
        self.master = {}  # key -> fp32 copy of a 16-bit shard

    def ensure_state(self, key, param):
        """[step, exp_avg, exp_avg_sq] of `key`, created (zero moments, fp32 master for a 16-bit shard) on first use."""
        return self._state(key, param)

    # ---- step constants on the device (for steps recorded as CUDA graphs)
    def use_device_scalars(self, device):
        """From now on the fused kernels read the step's constants from device memory: one counter and one set of
        constants shared by every key, advanced by advance_on_device() once per optimizer step."""
        if getattr(self, "_scalars_dev", None) is None:
            self._step_dev = torch.zeros(1, dtype=torch.float64, device=device)
            self._scalars_dev = torch.zeros(8, dtype=torch.float32, device=device)
            self.advance_on_device()  # the constants of step 1

    def device_scalars(self):
        return getattr(self, "_scalars_dev", None)

    def advance_on_device(self):
        from ..ops.elementwise import adam_prepare

        adam_prepare(self._step_dev, (self.lr, self.betas, self.eps, self.weight_decay), self._scalars_dev)

    def steps_on_device(self):
        """How many steps the device-side counter has prepared constants for, minus the one in preparation."""
        return float(self._step_dev.item()) - 1.0

    def _state(self, key, param):
        if key not in self.state:
            like = param if param.dtype in (torch.float32, torch.float64) else param.float()
            self.state[key] = [0.0, torch.zeros_like(like), torch.zeros_like(like)]
            if like is not param:
                self.master[key] = like  # param.float() made a fresh fp32 copy
        return self.state[key]

    def scalars(self, step):
        """(1 - lr*wd, 1 - beta1, beta2, 1 - beta2, sqrt(bias_correction2), eps, -lr / bias_correction1),
        computed in Python doubles exactly as torch does."""
        beta1, beta2 = self.betas
        bias1 = 1 - beta1 ** step
        bias2 = 1 - beta2 ** step
        return (1 - self.lr * self.weight_decay, 1 - beta1, beta2, 1 - beta2, bias2 ** 0.5, self.eps, -(self.lr / bias1))

    def update(self, key, param, grad, shadow=None):
        """One step for one shard.  `param` and `grad` have the same shape;
        `shadow`, if given, receives the updated parameter cast to its dtype."""
        st = self._state(key, param)
        st[0] += 1.0
        step, exp_avg, exp_avg_sq = st
        if param.numel() == 0:
            return
        master = self.master.get(key)
        if master is not None:  # 16-bit shard: step the fp32 master, write the shard back rounded
            if param.is_cuda and param.dtype == torch.bfloat16 and self.fused is not False:
                from ..ops import fused_adamw

                g = grad if grad.dtype in (torch.bfloat16, torch.float32) else grad.float()
                if self.device_scalars() is not None:
                    from ..ops.elementwise import adamw_step_dev

                    adamw_step_dev(master, g, exp_avg, exp_avg_sq, self._scalars_dev, param)
                else:
                    fused_adamw(master, g, exp_avg, exp_avg_sq, self.scalars(step), self.weight_decay != 0, param)
            else:
                self._torch_update(master, grad.float(), exp_avg, exp_avg_sq, step)
                param.copy_(master)
            if shadow is not None:
                shadow.copy_(param)
            return
        use_kernel = self.fused if self.fused is not None else (param.is_cuda and param.dtype == torch.float32)
        if use_kernel:
            from ..ops import fused_adamw

            if self.device_scalars() is not None and param.is_cuda:
                from ..ops.elementwise import adamw_step_dev

                adamw_step_dev(param, grad, exp_avg, exp_avg_sq, self._scalars_dev, shadow)
            else:
                fused_adamw(param, grad, exp_avg, exp_avg_sq, self.scalars(step), self.weight_decay != 0, shadow)
            return
        self._torch_update(param, grad, exp_avg, exp_avg_sq, step)
        if shadow is not None:
            shadow.copy_(param)

    def _torch_update(self, param, grad, exp_avg, exp_avg_sq, step):
        decay, w1, b2, w2, bias2_sqrt, eps, neg_step = self.scalars(step)
        if self.weight_decay != 0:
            param.mul_(decay)
        exp_avg.lerp_(grad, w1)
        exp_avg_sq.mul_(b2).addcmul_(grad, grad, value=w2)
        denom = (exp_avg_sq.sqrt() / bias2_sqrt).add_(eps)
        param.addcdiv_(exp_avg, denom, value=neg_step)

    def state_bytes(self):
        return sum(t.numel() * t.element_size() for _, m, v in self.state.values() for t in (m, v))

    # ---- checkpointing (layout: key -> {"step", "exp_avg", "exp_avg_sq"} of this rank's shard)
    def state_dict(self):
        return {"hyper": {"lr": self.lr, "betas": tuple(self.betas), "eps": self.eps, "weight_decay": self.weight_decay},
                "state": {k: {"step": s, "exp_avg": m.detach().cpu().clone(), "exp_avg_sq": v.detach().cpu().clone()}
                          for k, (s, m, v) in self.state.items()},
                "master": {k: t.detach().cpu().clone() for k, t in self.master.items()}}

    def load_state_dict(self, sd, device=None):
        h = sd["hyper"]
        self.lr, self.betas, self.eps, self.weight_decay = h["lr"], tuple(h["betas"]), h["eps"], h["weight_decay"]
        self.state = {}
        for k, e in sd["state"].items():
            dev = device if device is not None else e["exp_avg"].device
            self.state[k] = [float(e["step"]), e["exp_avg"].to(dev).clone(), e["exp_avg_sq"].to(dev).clone()]
        self.master = {k: t.to(device if device is not None else t.device).clone() for k, t in sd.get("master", {}).items()}
