"""Baseline optimizers selectable through `--opt`: Lion, Signum / signSGD, ADOPT, LAMB, Adafactor,
Prodigy, Sophia-G, MARS (AdamW / Lion variants), schedule-free AdamW / SGD and SOAP.

These are the comparison points of the reference (src/optim/{lion,sign,adopt,lamb,adafactor,prodigy,
sophia,mars,schedulefree,soap}.py); they are written here from the published algorithms as compact
per-tensor PyTorch optimizers and are not on the kernel path.  Each keeps the hooks the training loop
relies on: schedule-free `.train()/.eval()`, Sophia `.update_hessian()` and `step(bs=...)`, MARS
`.update_last_grad()`, Prodigy's `d`, `k`, `use_bias_correction` group entries.
"""
from __future__ import annotations

import math

import torch
from torch.optim import Optimizer


class Lion(Optimizer):
    """update = sign(b1 m + (1-b1) g); m <- b2 m + (1-b2) g; decoupled weight decay."""

    def __init__(self, params, lr=1e-4, betas=(0.9, 0.99), weight_decay=0.0):
        super().__init__(params, dict(lr=lr, betas=betas, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self, closure=None):
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["exp_avg"] = torch.zeros_like(p)
                p.mul_(1 - g["lr"] * g["weight_decay"])
                upd = st["exp_avg"].mul(b1).add_(p.grad, alpha=1 - b1).sign_()
                p.add_(upd, alpha=-g["lr"])
                st["exp_avg"].mul_(b2).add_(p.grad, alpha=1 - b2)


class Signum(Optimizer):
    """SGD on the sign of the (momentum-averaged) gradient; momentum 0 gives signSGD."""

    def __init__(self, params, lr=1e-3, momentum=0.0, dampening=0.0, weight_decay=0.0, nesterov=False,
                 sign_update=True):
        if nesterov and (momentum <= 0 or dampening != 0):
            raise ValueError("Nesterov momentum requires a momentum and zero dampening")
        super().__init__(params, dict(lr=lr, momentum=momentum, dampening=dampening, weight_decay=weight_decay,
                                      nesterov=nesterov, sign_update=sign_update))

    @torch.no_grad()
    def step(self, closure=None):
        for g in self.param_groups:
            mu = g["momentum"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                d = p.grad
                p.mul_(1 - g["lr"] * g["weight_decay"])
                st = self.state[p]
                st["step"] = st.get("step", 0) + 1
                if mu != 0:
                    if "momentum_buffer" not in st:
                        # as in the reference (src/optim/sign.py:43-52): the buffer starts as a copy of the
                        # (already decayed) PARAMETER, not of the gradient, and is averaged from the first step on
                        st["momentum_buffer"] = p.detach().clone()
                    buf = st["momentum_buffer"].mul_(mu).add_(d, alpha=1 - g["dampening"])
                    d = d.add(buf, alpha=mu) if g["nesterov"] else buf
                p.add_(d.sign() if g["sign_update"] else d, alpha=-g["lr"])


class ADOPT(Optimizer):
    """Adam with the second moment of the PREVIOUS step in the denominator (no bias correction)."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.9999), eps=1e-6, weight_decay=0.0, decouple=True):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, decouple=decouple))

    @torch.no_grad()
    def step(self, closure=None):
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                grad = p.grad
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(p)
                    st["exp_avg_sq"] = grad * grad
                    st["step"] = 1
                    continue
                if g["weight_decay"] != 0:
                    if g["decouple"]:
                        p.mul_(1 - g["lr"] * g["weight_decay"])
                    else:
                        grad = grad.add(p, alpha=g["weight_decay"])
                denom = st["exp_avg_sq"].sqrt().clamp_(min=g["eps"])
                normed = grad / denom
                clip = st["step"] ** 0.25
                normed.clamp_(-clip, clip)
                st["exp_avg"].lerp_(normed, 1 - b1)
                p.add_(st["exp_avg"], alpha=-g["lr"])
                st["exp_avg_sq"].mul_(b2).addcmul_(grad, grad, value=1 - b2)
                st["step"] += 1


class Lamb(Optimizer):
    """Adam direction rescaled per tensor by ||w|| / ||update||."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-6, weight_decay=0.0, adam=False, bias_correction=False):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self.adam, self.bias_correction = adam, bias_correction

    @torch.no_grad()
    def step(self, closure=None):
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(p)
                    st["exp_avg_sq"] = torch.zeros_like(p)
                st["step"] += 1
                st["exp_avg"].mul_(b1).add_(p.grad, alpha=1 - b1)
                st["exp_avg_sq"].mul_(b2).addcmul_(p.grad, p.grad, value=1 - b2)
                m, v = st["exp_avg"], st["exp_avg_sq"]
                if self.bias_correction:
                    m = m / (1 - b1 ** st["step"])
                    v = v / (1 - b2 ** st["step"])
                upd = m / (v.sqrt() + g["eps"])
                if g["weight_decay"] != 0:
                    upd = upd.add(p, alpha=g["weight_decay"])
                wn, un = p.norm().clamp(0, 10), upd.norm()
                trust = 1.0 if (self.adam or wn == 0 or un == 0) else (wn / un).item()
                st["trust_ratio"] = trust
                p.add_(upd, alpha=-g["lr"] * trust)


class Adafactor(Optimizer):
    """Factored second moments for matrices (row and column statistics), update clipping, optional momentum.

    Defaults follow the reference (src/optim/adafactor.py:57-110), including the ones that make `lr` a no-op there:
    with `relative_step` the step size is min(1e-2, 1/sqrt(t)) (or 1e-6 t with `warmup_init`), with `scale_parameter`
    it is multiplied by max(eps2[1], RMS(parameter)); momentum averages the already scaled update and the decoupled
    weight decay uses the same step size."""

    def __init__(self, params, lr=1e-3, eps2=(1e-30, 1e-3), clip_threshold=1.0, decay_rate=-0.8, beta1=None,
                 weight_decay=0.0, scale_parameter=True, relative_step=True, warmup_init=False):
        super().__init__(params, dict(lr=lr, eps2=eps2, clip_threshold=clip_threshold, decay_rate=decay_rate, beta1=beta1,
                                      weight_decay=weight_decay, scale_parameter=scale_parameter,
                                      relative_step=relative_step, warmup_init=warmup_init))

    @staticmethod
    def _rms(t):
        return t.norm(2) / (t.numel() ** 0.5)

    @torch.no_grad()
    def step(self, closure=None):
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                grad = p.grad
                st = self.state[p]
                factored = grad.dim() >= 2
                if not st:
                    st["step"] = 0
                    if factored:
                        st["exp_avg_sq_row"] = torch.zeros(grad.shape[:-1], device=grad.device, dtype=grad.dtype)
                        st["exp_avg_sq_col"] = torch.zeros(grad.shape[:-2] + grad.shape[-1:], device=grad.device,
                                                           dtype=grad.dtype)
                    else:
                        st["exp_avg_sq"] = torch.zeros_like(grad)
                    if g["beta1"] is not None:
                        st["exp_avg"] = torch.zeros_like(grad)
                st["step"] += 1
                st["RMS"] = self._rms(p)
                step_size = g["lr"]
                if g["relative_step"]:
                    floor = 1e-6 * st["step"] if g["warmup_init"] else 1e-2
                    step_size = min(floor, 1.0 / math.sqrt(st["step"]))
                if g["scale_parameter"]:
                    step_size = step_size * max(g["eps2"][1], st["RMS"])
                rho = 1.0 - math.pow(st["step"], g["decay_rate"])
                sq = grad * grad + g["eps2"][0]
                if factored:
                    row, col = st["exp_avg_sq_row"], st["exp_avg_sq_col"]
                    row.mul_(rho).add_(sq.mean(-1), alpha=1.0 - rho)
                    col.mul_(rho).add_(sq.mean(-2), alpha=1.0 - rho)
                    r = (row / row.mean(-1)).rsqrt_().unsqueeze(-1)
                    upd = (r * col.unsqueeze(-2).rsqrt()).mul_(grad)
                else:
                    st["exp_avg_sq"].mul_(rho).add_(sq, alpha=1.0 - rho)
                    upd = st["exp_avg_sq"].rsqrt().mul_(grad)
                upd.div_(max(1.0, self._rms(upd) / g["clip_threshold"]))
                upd.mul_(step_size)
                if g["beta1"] is not None:
                    upd = st["exp_avg"].mul_(g["beta1"]).add_(upd, alpha=1 - g["beta1"])
                if g["weight_decay"] != 0:
                    p.add_(p, alpha=-g["weight_decay"] * step_size)
                p.add_(-upd)


class Prodigy(Optimizer):
    """Adam whose step-size scale d is estimated on the fly from <g, x0 - x> / ||s|| (parameter-free)."""

    def __init__(self, params, lr=1.0, betas=(0.9, 0.999), beta3=None, eps=1e-8, weight_decay=0.0, decouple=True,
                 use_bias_correction=False, safeguard_warmup=False, d0=1e-6, d_coef=1.0, growth_rate=float("inf"),
                 fsdp_in_use=False):
        super().__init__(params, dict(lr=lr, betas=betas, beta3=beta3, eps=eps, weight_decay=weight_decay, d=d0, d0=d0,
                                      d_max=d0, d_numerator=0.0, d_coef=d_coef, k=0, growth_rate=growth_rate,
                                      use_bias_correction=use_bias_correction, decouple=decouple,
                                      safeguard_warmup=safeguard_warmup, fsdp_in_use=fsdp_in_use))

    @torch.no_grad()
    def step(self, closure=None):
        g0 = self.param_groups[0]
        b1, b2 = g0["betas"]
        b3 = g0["beta3"] if g0["beta3"] is not None else math.sqrt(b2)
        k, d, d_max, d0, lr = g0["k"], g0["d"], g0["d_max"], g0["d0"], max(g["lr"] for g in self.param_groups)
        bias = ((1 - b2 ** (k + 1)) ** 0.5) / (1 - b1 ** (k + 1)) if g0["use_bias_correction"] else 1.0
        dlr = d * lr * bias
        num = g0["d_numerator"] * b3
        num_acc = torch.zeros((), device=self.param_groups[0]["params"][0].device)
        den_acc = torch.zeros_like(num_acc)
        sharded = False
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                grad = p.grad
                st = self.state[p]
                if not st:
                    st["s"] = torch.zeros_like(p)
                    st["p0"] = p.detach().clone()
                    st["exp_avg"] = torch.zeros_like(p)
                    st["exp_avg_sq"] = torch.zeros_like(p)
                if g["weight_decay"] != 0 and not g["decouple"]:
                    grad = grad.add(p, alpha=g["weight_decay"])
                if lr > 0:
                    # (sharded parameters: each rank adds what its shard contributes; the sums meet in the all-reduce below)
                    loc = lambda t: t.to_local() if hasattr(t, "to_local") else t
                    sharded = sharded or hasattr(p, "to_local")
                    num_acc += (d / d0) * dlr * torch.dot(loc(grad).flatten(), loc(st["p0"] - p).flatten())
                    st["exp_avg"].mul_(b1).add_(grad, alpha=d * (1 - b1))
                    st["exp_avg_sq"].mul_(b2).addcmul_(grad, grad, value=d * d * (1 - b2))
                    alpha = (d / d0) * (d if g["safeguard_warmup"] else dlr)
                    st["s"].mul_(b3).add_(grad, alpha=alpha)
                    den_acc += loc(st["s"]).abs().sum()
        if (g0["fsdp_in_use"] or sharded) and torch.distributed.is_initialized():
            both = torch.stack([num_acc, den_acc])
            torch.distributed.all_reduce(both)
            num_acc, den_acc = both[0], both[1]
        d_hat = d
        if lr > 0 and float(den_acc) > 0:
            num = num + float(num_acc)
            d_hat = g0["d_coef"] * num / float(den_acc)
            if d == d0:
                d = max(d, d_hat)
            d_max = max(d_max, d_hat)
            d = min(d_max, d * g0["growth_rate"])
        for g in self.param_groups:
            g.update(d_numerator=num, d=d, d_max=d_max, d_hat=d_hat, k=k + 1)
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                denom = st["exp_avg_sq"].sqrt().add_(d * g["eps"])
                if g["weight_decay"] != 0 and g["decouple"]:
                    p.add_(p, alpha=-g["weight_decay"] * dlr)
                p.addcdiv_(st["exp_avg"], denom, value=-dlr)


class SophiaG(Optimizer):
    """Clipped second-order step m / max(rho * bs * h, eps) with a Gauss-Newton-Bartlett Hessian EMA."""

    def __init__(self, params, lr=1e-4, betas=(0.965, 0.99), rho=0.04, weight_decay=1e-1):
        super().__init__(params, dict(lr=lr, betas=betas, rho=rho, weight_decay=weight_decay))

    def _init(self, p):
        st = self.state[p]
        if not st:
            st["step"] = 0
            st["exp_avg"] = torch.zeros_like(p)
            st["hessian"] = torch.zeros_like(p)
        return st

    @torch.no_grad()
    def update_hessian(self):
        for g in self.param_groups:
            b2 = g["betas"][1]
            for p in g["params"]:
                if p.grad is not None:
                    self._init(p)["hessian"].mul_(b2).addcmul_(p.grad, p.grad, value=1 - b2)

    @torch.no_grad()
    def step(self, closure=None, bs=5120):
        for g in self.param_groups:
            b1 = g["betas"][0]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self._init(p)
                st["step"] += 1
                st["exp_avg"].mul_(b1).add_(p.grad, alpha=1 - b1)
                p.mul_(1 - g["lr"] * g["weight_decay"])
                ratio = (st["exp_avg"].abs() / (g["rho"] * bs * st["hessian"] + 1e-15)).clamp_(max=1.0)
                p.addcmul_(st["exp_avg"].sign(), ratio, value=-g["lr"])


class MARS(Optimizer):
    """Variance-reduced gradient c_t = g_t + gamma * b1/(1-b1) * (g_t - g_{t-1}) (norm-clipped to 1) fed to AdamW or
    Lion for >=2-D tensors; 1-D tensors use plain AdamW with their own lr / betas unless `optimize_1d`."""

    def __init__(self, params, lr=3e-3, betas=(0.95, 0.99), eps=1e-8, weight_decay=0.0, amsgrad=False, gamma=0.025,
                 is_approx=True, mars_type="mars-adamw", optimize_1d=False, lr_1d=3e-3, betas_1d=(0.9, 0.95),
                 weight_decay_1d=0.1):
        if mars_type not in ("mars-adamw", "mars-lion", "mars-shampoo"):
            raise ValueError(mars_type)
        # the same group keys as the reference (src/optim/mars.py:141-163), so that `state_dict()`s interchange; the
        # approximation switch and the 1-D learning rate / betas are attributes there and here
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, amsgrad=amsgrad,
                                      mars_type=mars_type, gamma=gamma, optimize_1d=optimize_1d,
                                      weight_decay_1d=weight_decay_1d))
        self.is_approx, self.betas_1d = is_approx, betas_1d
        # the 1-D tensors follow the schedule too: their rate is the group's current lr times this constant ratio
        # (src/optim/mars.py:163, 84-86)
        self.lr_1d_factor = lr_1d / lr

    @torch.no_grad()
    def update_last_grad(self):
        """The exact variant re-evaluates the previous batch; the approximate one reuses the stored gradient."""
        for g in self.param_groups:
            for p in g["params"]:
                st = self.state.get(p)
                if st and "pending_last" in st:
                    st["last_grad"] = st.pop("pending_last")

    @torch.no_grad()
    def step(self, closure=None):
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                grad = p.grad
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(p)
                    st["exp_avg_sq"] = torch.zeros_like(p)
                    st["last_grad"] = torch.zeros_like(p)
                st["step"] += 1
                t = st["step"]
                if p.dim() == 2 or g["optimize_1d"]:
                    c = grad + g["gamma"] * (b1 / (1 - b1)) * (grad - st["last_grad"])
                    n = c.norm()
                    if n > 1.0:
                        c = c / n
                    st["exp_avg"].mul_(b1).add_(c, alpha=1 - b1)
                    if g["mars_type"] == "mars-lion":
                        upd = st["exp_avg"].sign()
                    elif g["mars_type"] == "mars-shampoo" and p.dim() == 2:
                        from .muon import newton_schulz5

                        upd = newton_schulz5(st["exp_avg"], steps=5) * max(1, p.size(0) / p.size(1)) ** 0.5
                    else:
                        st["exp_avg_sq"].mul_(b2).addcmul_(c, c, value=1 - b2)
                        upd = (st["exp_avg"] / (1 - b1 ** t)) / ((st["exp_avg_sq"] / (1 - b2 ** t)).sqrt() + g["eps"])
                    p.mul_(1 - g["lr"] * g["weight_decay"])
                    p.add_(upd, alpha=-g["lr"])
                else:
                    c1, c2 = self.betas_1d
                    st["exp_avg"].mul_(c1).add_(grad, alpha=1 - c1)
                    st["exp_avg_sq"].mul_(c2).addcmul_(grad, grad, value=1 - c2)
                    upd = (st["exp_avg"] / (1 - c1 ** t)) / ((st["exp_avg_sq"] / (1 - c2 ** t)).sqrt() + g["eps"])
                    lr_1d = g["lr"] * self.lr_1d_factor
                    p.mul_(1 - lr_1d * g["weight_decay_1d"])
                    p.add_(upd, alpha=-lr_1d)
                st["pending_last"] = grad.detach().clone()
                if self.is_approx:
                    st["last_grad"] = st["pending_last"]


class _ScheduleFree(Optimizer):
    """Schedule-free base: gradients are taken at y = (1-b) z + b x, z takes the raw step and x is the
    c_t-weighted average of z; `.eval()` swaps the parameters to x, `.train()` back to y."""

    def __init__(self, params, defaults):
        # as in the reference (src/optim/schedulefree.py:66-79): not in train mode until `.train()` is called
        defaults.update(train_mode=False, k=0, weight_sum=0.0, lr_max=-1.0, scheduled_lr=0.0)
        super().__init__(params, defaults)

    def _beta(self, g):
        raise NotImplementedError

    @torch.no_grad()
    def _swap(self, to_train: bool):
        for g in self.param_groups:
            if g["train_mode"] == to_train:
                continue
            b = self._beta(g)
            for p in g["params"]:
                st = self.state.get(p)
                if st and "z" in st:
                    # y = (1-b) z + b x  <=>  x = (y - (1-b) z) / b
                    if to_train:
                        p.lerp_(st["z"], 1 - b)
                    else:
                        p.lerp_(st["z"], 1 - 1 / b)
            g["train_mode"] = to_train

    def train(self):
        self._swap(True)

    def eval(self):
        self._swap(False)

    def _require_train_mode(self):
        if not self.param_groups[0]["train_mode"]:
            raise RuntimeError("Optimizer was not in train mode when step is called: call .train() before training "
                               "steps and .eval() before evaluation or checkpointing")

    def _schedule(self, g):
        k = g["k"]
        sched = (k + 1) / g["warmup_steps"] if k < g["warmup_steps"] else 1.0
        return sched

    def _weights(self, g, lr):
        g["lr_max"] = max(lr, g["lr_max"])
        w = ((g["k"] + 1) ** g["r"]) * (g["lr_max"] ** g["weight_lr_power"])
        g["weight_sum"] += w
        return w / g["weight_sum"] if g["weight_sum"] > 0 else 0.0


class AdamWScheduleFree(_ScheduleFree):
    def __init__(self, params, lr=0.0025, betas=(0.9, 0.999), eps=1e-8, weight_decay=0, warmup_steps=0, r=0.0,
                 weight_lr_power=2.0):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, warmup_steps=warmup_steps,
                                      r=r, weight_lr_power=weight_lr_power))

    def _beta(self, g):
        return g["betas"][0]

    @torch.no_grad()
    def step(self, closure=None):
        self._require_train_mode()
        for g in self.param_groups:
            b1, b2 = g["betas"]
            bc2 = 1 - b2 ** (g["k"] + 1)
            # the reference's variant (src/optim/schedulefree.py:137-190): the bias correction sits inside the
            # denominator, sqrt(v / bc2) + eps, and the step size is not rescaled by it
            lr = g["scheduled_lr"] = g["lr"] * self._schedule(g)
            ck = self._weights(g, lr)
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if "z" not in st:
                    st["z"] = p.detach().clone()
                    st["exp_avg_sq"] = torch.zeros_like(p)
                st["exp_avg_sq"].mul_(b2).addcmul_(p.grad, p.grad, value=1 - b2)
                gn = p.grad / (st["exp_avg_sq"].div(bc2).sqrt_().add_(g["eps"]))
                if g["weight_decay"] != 0:
                    gn.add_(p, alpha=g["weight_decay"])
                p.lerp_(st["z"], ck)                       # y moves towards z as x does
                p.add_(gn, alpha=lr * (b1 * (1 - ck) - 1))
                st["z"].sub_(gn, alpha=lr)
            g["k"] += 1


class SGDScheduleFree(_ScheduleFree):
    def __init__(self, params, lr=1.0, momentum=0.9, weight_decay=0, warmup_steps=0, r=0.0, weight_lr_power=2.0):
        super().__init__(params, dict(lr=lr, momentum=momentum, weight_decay=weight_decay, warmup_steps=warmup_steps,
                                      r=r, weight_lr_power=weight_lr_power))

    def _beta(self, g):
        return g["momentum"]

    @torch.no_grad()
    def step(self, closure=None):
        self._require_train_mode()
        for g in self.param_groups:
            b = g["momentum"]
            lr = g["scheduled_lr"] = g["lr"] * self._schedule(g)
            ck = self._weights(g, lr)
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if "z" not in st:
                    st["z"] = p.detach().clone()
                grad = p.grad if g["weight_decay"] == 0 else p.grad.add(p, alpha=g["weight_decay"])
                p.lerp_(st["z"], ck)
                p.add_(grad, alpha=lr * (b * (1 - ck) - 1))
                st["z"].sub_(grad, alpha=lr)
            g["k"] += 1


class SOAP(Optimizer):
    """Adam run in the eigenbasis of Shampoo's Kronecker-factor statistics; the basis is refreshed every
    `precondition_frequency` steps with one QR power-iteration step."""

    def __init__(self, params, lr=3e-3, betas=(0.95, 0.95), shampoo_beta=-1.0, eps=1e-8, weight_decay=0.01,
                 precondition_frequency=10, max_precond_dim=10000, merge_dims=False, precondition_1d=False,
                 normalize_grads=False, data_format="channels_first", correct_bias=True):
        super().__init__(params, dict(lr=lr, betas=betas, shampoo_beta=shampoo_beta, eps=eps, weight_decay=weight_decay,
                                      precondition_frequency=precondition_frequency, max_precond_dim=max_precond_dim,
                                      merge_dims=merge_dims, precondition_1d=precondition_1d,
                                      normalize_grads=normalize_grads, correct_bias=correct_bias))

    @staticmethod
    def _project(x, Q, back=False):
        for i, q in enumerate(Q):
            if q is None:
                x = x.movedim(0, -1)
                continue
            x = torch.tensordot(x, q if not back else q.T, dims=([0], [0]))
        return x

    @torch.no_grad()
    def step(self, closure=None):
        for g in self.param_groups:
            b1, b2 = g["betas"]
            sb = g["shampoo_beta"] if g["shampoo_beta"] >= 0 else b2
            for p in g["params"]:
                if p.grad is None:
                    continue
                grad = p.grad.float()
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(grad)
                    st["exp_avg_sq"] = torch.zeros_like(grad)
                    use = grad.dim() >= 2 or g["precondition_1d"]
                    st["GG"] = [torch.zeros(s, s, device=grad.device) if (use and s <= g["max_precond_dim"]) else None
                                for s in grad.shape]
                    st["Q"] = None
                for i, gg in enumerate(st["GG"]):
                    if gg is not None:
                        other = [d for d in range(grad.dim()) if d != i]
                        gg.lerp_(torch.tensordot(grad, grad, dims=(other, other)), 1 - sb)
                if st["Q"] is None:
                    st["Q"] = [None if gg is None else torch.linalg.eigh(gg + 1e-30 * torch.eye(gg.shape[0], device=gg.device))[1].flip(1)
                               for gg in st["GG"]]
                    continue                                  # the first step only builds the basis
                st["step"] += 1
                gp = self._project(grad, st["Q"])
                st["exp_avg"].mul_(b1).add_(grad, alpha=1 - b1)
                st["exp_avg_sq"].mul_(b2).addcmul_(gp, gp, value=1 - b2)
                mp = self._project(st["exp_avg"], st["Q"])
                step_size = g["lr"]
                if g["correct_bias"]:
                    step_size *= math.sqrt(1 - b2 ** st["step"]) / (1 - b1 ** st["step"])
                upd = self._project(mp / (st["exp_avg_sq"].sqrt() + g["eps"]), st["Q"], back=True)
                if g["normalize_grads"]:
                    upd = upd / (1e-30 + upd.pow(2).mean().sqrt())
                p.add_(upd.to(p.dtype), alpha=-step_size)
                if g["weight_decay"] > 0:
                    p.mul_(1 - g["lr"] * g["weight_decay"])
                if st["step"] % g["precondition_frequency"] == 0:
                    # rotate the second moment back, refresh the basis by one orthogonal-iteration step
                    v_full = self._project(st["exp_avg_sq"], st["Q"], back=True)
                    new_q = []
                    for gg, q in zip(st["GG"], st["Q"]):
                        if gg is None:
                            new_q.append(None)
                            continue
                        est = torch.diag(q.T @ gg @ q)
                        order = torch.argsort(est, descending=True)
                        new_q.append(torch.linalg.qr(gg @ q[:, order])[0])
                    st["Q"] = new_q
                    st["exp_avg_sq"] = self._project(v_full, st["Q"]).abs_()


def build(name, args, group_specs):
    b = (args.beta1, args.beta2)
    if name == "lion":
        return Lion(group_specs, lr=args.lr, betas=b, weight_decay=args.weight_decay)
    if name in ("signsgd", "signum"):
        mom = 0.0 if name == "signsgd" else args.momentum
        return Signum(group_specs, lr=args.lr, momentum=mom, dampening=args.dampening, weight_decay=args.weight_decay,
                      nesterov=bool(args.nesterov) and mom > 0, sign_update=True)
    if name == "adopt":
        return ADOPT(group_specs, lr=args.lr, betas=b, eps=args.adopt_eps, weight_decay=args.weight_decay,
                     decouple=args.adopt_decouple)
    if name == "lamb":
        return Lamb(group_specs, lr=args.lr, betas=b, weight_decay=args.weight_decay, adam=False,
                    bias_correction=args.lamb_use_bias_correction)
    if name == "adafactor":
        return Adafactor(group_specs, lr=args.lr, decay_rate=args.adafactor_decay_rate, beta1=args.beta1,
                         clip_threshold=1.0, weight_decay=args.weight_decay)
    if name == "prodigy":
        return Prodigy(group_specs, lr=args.lr, betas=b, beta3=args.prodigy_beta3, weight_decay=args.weight_decay,
                       decouple=args.prodigy_decouple, use_bias_correction=args.prodigy_use_bias_correction,
                       safeguard_warmup=args.prodigy_safeguard_warmup, fsdp_in_use=args.prodigy_fsdp_in_use)
    if name == "sophiag":
        return SophiaG(group_specs, lr=args.lr, betas=b, weight_decay=args.weight_decay, rho=args.sophia_rho)
    if name == "mars":
        return MARS(group_specs, lr=args.mars_lr, betas=(args.mars_beta1, args.mars_beta2), weight_decay=args.weight_decay,
                    gamma=args.mars_vr_gamma, is_approx=args.mars_is_approx, mars_type=args.mars_type, optimize_1d=False,
                    lr_1d=args.lr, betas_1d=b, weight_decay_1d=0.1)
    if name == "sf-adamw":
        return AdamWScheduleFree(group_specs, lr=args.lr, betas=b, weight_decay=args.weight_decay,
                                 warmup_steps=args.warmup_steps, r=args.schedulefree_r, weight_lr_power=args.weight_lr_power)
    if name == "sf-sgd":
        return SGDScheduleFree(group_specs, lr=args.lr, momentum=args.momentum, weight_decay=args.weight_decay,
                               warmup_steps=args.warmup_steps, r=args.schedulefree_r, weight_lr_power=args.weight_lr_power)
    if name == "soap":
        return SOAP(group_specs, lr=args.lr, betas=b, shampoo_beta=args.shampoo_beta, weight_decay=args.weight_decay,
                    precondition_frequency=args.precondition_frequency, max_precond_dim=args.max_precond_dim,
                    merge_dims=args.merge_dims, precondition_1d=args.precondition_1d,
                    normalize_grads=args.normalize_grads, data_format=args.soap_data_format,
                    correct_bias=args.correct_bias)
    raise ValueError(f"Unknown optimizer: '{name}'")
