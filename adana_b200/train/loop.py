"""Training runtime: the step loop, evaluation, checkpoint cadence and logging.

`train(model, opt, datareaders, scheduler, exp_dir, distributed_backend, cfg) -> stats` keeps
the reference's contract (src/optim/base.py:25-362): per iteration it may write a permanent
and/or `latest` checkpoint, evaluates every `eval_interval`, stops cleanly after
`iterations_to_run` (writing `latest` first), runs `acc_steps` micro-steps, clips, steps the
optimizer and scheduler and prints

    Train: Iter=<i> (<e> epochs) train_loss=<l> iter_dt=<s>s lr=<lr>
    >Eval: Iter=<i> (<e> epochs) val_loss=<l> val_pp=<p> val_acc=<a>
    [Memory] GPU 0: peak_allocated=<x> GiB, peak_reserved=<y> GiB
    [Checkpoint] START|END ...

(the formats scripts grep for).  Differences: the loop is a `Trainer` object with one method per
phase; `iter_dt` can be measured on the device with CUDA events (max over ranks,
`--device_timing`) instead of host time without a sync; batches go through a pinned staging
buffer with asynchronous host-to-device copies; NVTX ranges mark the phases (`--nvtx`); a
host-side heartbeat watchdog can abort a rank whose peers stopped responding
(`--heartbeat_timeout`).
"""
from __future__ import annotations

import contextlib
import copy
import os
import time
from contextlib import nullcontext
from pathlib import Path

import torch
import torch.distributed as dist

from ..data.readers import PinnedBatchStager
from ..utils.timing import DeviceTimer, nvtx_range
from . import checkpoint as ckpt

try:  # optional
    import wandb
except Exception:  # pragma: no cover
    wandb = None


def get_batch(reader, device="cpu"):
    """Pinned host buffer + non-blocking copy of one batch (PyTorch-path helper)."""
    x, y = reader.sample_batch()
    if "cuda" in str(device):
        x = x.pin_memory().to(device, non_blocking=True)
        y = y.pin_memory().to(device, non_blocking=True)
    else:
        x, y = x.to(device), y.to(device)
    return x, y


@torch.no_grad()
def evaluate(model, reader, device="cpu", max_num_batches=24, ctx=nullcontext(), moe=False,
             get_router_logits=False, cfg=None):
    assert not model.training
    losses, accs, aux, router = [], [], {}, []
    for _ in range(max_num_batches):
        x, y = get_batch(reader, device=device)
        with ctx:
            out = model(x, targets=y, get_logits=False, moe=moe, compute_accuracy=True)
        losses.append(out["loss"].detach().float())
        accs.append(out["accuracy"].float())
        for k, v in out["aux_losses"].items():
            aux.setdefault(k, []).append(torch.as_tensor(v).detach().float())
        if get_router_logits and out["router_logits"] is not None:
            router.append(out["router_logits"])
    val_loss = torch.stack(losses).mean().item()
    val_acc = torch.stack(accs).mean().item()
    val_aux = {f"val/{k}": torch.stack(v).mean().item() for k, v in aux.items()}
    if get_router_logits and router:
        size = (cfg.batch_size * cfg.sequence_length) if cfg else router[0].shape[1]
        router = torch.stack([r for r in router if r.shape[1] == size], 0).detach().cpu()
    return val_acc, val_loss, 2.71828 ** val_loss, val_aux, router


class Trainer:
    def __init__(self, model, opt, datareaders, scheduler, exp_dir, backend, cfg):
        self.model, self.opt, self.scheduler = model, opt, scheduler
        self.exp_dir, self.backend, self.cfg = Path(exp_dir), backend, cfg
        self.train_reader, self.val_reader = datareaders["train"], datareaders["val"]
        self.master = backend.is_master_process()
        self.all_ranks_ckpt = backend.all_ranks_checkpoint()
        self.engine = getattr(backend, "engine", None)
        self.cuda = "cuda" in str(cfg.device)
        self.type_ctx = nullcontext()
        if self.cuda and (self.engine is None):
            dt = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}[cfg.dtype]
            self.type_ctx = torch.amp.autocast(device_type="cuda", dtype=dt)
        self.run_model = model
        if cfg.compile and self.engine is None:
            print("Compiling model ...")
            self.run_model = torch.compile(model)
        self.stager = PinnedBatchStager(self.train_reader, cfg.device, lookahead=False)
        self.timer = DeviceTimer(enabled=self.cuda and getattr(cfg, "device_timing", False))
        self.stats = {"train_loss": [], "val_loss": [], "val_pp": [], "val_acc": []}
        self.grad_norms = []
        self.curr_iter = 0
        self.substep = 0
        self.iters_in_run = 0
        self.tau_stats = None
        self.dlogger = None
        self.watchdog = None
        # expert-parallel layers exchange tokens between the ranks inside every forward: no rank can evaluate alone
        self.collective_forward = any(getattr(p, "_adana_rank_local", False) for p in self.model.parameters())
        # Host-side fault injection for the recovery tests: ADANA_FAULT_EXIT="<rank>:<iteration>[:<exit code>]" makes
        # that rank leave the job at the top of that iteration, between steps, with nothing of its own in flight.
        self._exit_at = None
        spec = os.environ.get("ADANA_FAULT_EXIT")
        if spec:
            parts = spec.split(":")
            rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
            if int(parts[0]) == rank:
                self._exit_at = (int(parts[1]), int(parts[2]) if len(parts) > 2 else 17)

    # ---- set-up ---------------------------------------------------------------------------------------
    def setup(self):
        cfg = self.cfg
        if cfg.resume_from:
            print(f"\nResuming Training From {cfg.resume_from}")
            d = Path(cfg.resume_from)
            self.curr_iter = ckpt.load_checkpoint(self.model, self.opt, self.scheduler, d / "main.pt",
                                                  cfg.device, distributed_backend=self.backend)
            ckpt.load_worker_state(d, train_reader=self.train_reader)
            self.substep = self.curr_iter * cfg.acc_steps
        else:
            self.train_reader.set_step(0)
        from ..logging.metrics import MetricsSink

        self.sink = MetricsSink(self.exp_dir, wandb if (cfg.wandb and wandb is not None) else None, enabled=self.master)
        counts = getattr(self.backend, "param_counts", None)
        if counts is not None:      # the first record of a run, as in the reference (src/main.py:376-379)
            self.sink.log({"parameters": counts[0], "optimized_parameters": counts[1]})
        engine = getattr(self.backend.get_raw_model(self.model), "_engine", None)
        gathers = engine is not None and engine.sharded and engine.world > 1   # then every rank takes part
        if getattr(cfg, "log_dynamics", False) and (self.master or gathers):
            from ..logging.dynamics import DynamicsLogger, load_logger_config

            self.dlogger = DynamicsLogger(self.model, self.opt, load_logger_config(cfg.dynamics_logger_cfg),
                                          self.exp_dir, wandb=cfg.wandb and self.master, write=self.master)
            self.dlogger.iteration = self.curr_iter
        if self.master and getattr(cfg, "collect_tau_stats", False) and cfg.opt in ("dana-star-mk4", "dana-star"):
            from ..logging.tau_stats import TauStatsCollector

            names = [n for g in self.opt.param_groups for n in g.get("param_names", [])]
            self.tau_stats = TauStatsCollector(exp_dir=self.exp_dir, cfg=cfg, param_names=names)
        hb = float(getattr(cfg, "heartbeat_timeout", 0.0) or 0.0)
        if hb > 0 and dist.is_available() and dist.is_initialized():
            from ..runtime.watchdog import HeartbeatWatchdog

            self.watchdog = HeartbeatWatchdog.from_env(timeout_s=hb)
            self.watchdog.start()
        self.model.train()

    # ---- device status word ------------------------------------------------------------------------------
    def _read_device_status(self):
        """Raises when a kernel of this process recorded a timed-out wait (a late or dead peer, a stuck pipeline)
        in the device status word.  Synchronises the device, so it is called only where the loop synchronises
        anyway: on logging iterations, before a checkpoint is written and at the end of the run."""
        if self.cuda and self.engine is not None:
            from ..ops import _lib

            _lib.check_status(self.cfg.device)

    def check_device_status(self):
        try:
            self._read_device_status()
        except RuntimeError as e:
            # after a timed-out wait the gradients and weights of this step may be built on stale peer data: stop
            # here, before they are logged as progress or written to a checkpoint
            raise RuntimeError(f"iteration {self.curr_iter}: {e}; the run stops before this state is checkpointed") from e

    def _phase(self, name):
        return self.watchdog.phase(name) if self.watchdog is not None else contextlib.nullcontext()

    # ---- checkpoints ------------------------------------------------------------------------------------
    def _write_checkpoint(self, ckpt_dir: Path, label: str):
        with self._phase("checkpoint"):
            self.check_device_status()
            self._write_checkpoint_files(ckpt_dir, label)

    def _write_checkpoint_files(self, ckpt_dir: Path, label: str):
        cfg = self.cfg
        if self.master:
            print(f"[Checkpoint] START {label} iter={self.curr_iter} -> {ckpt_dir}")
        if self.master or self.all_ranks_ckpt:
            ckpt.save_checkpoint(self.model, self.opt, self.scheduler, self.curr_iter, ckpt_dir,
                                 distributed_backend=self.backend,
                                 async_write=getattr(cfg, "async_checkpoint", False))
        if self.master and cfg.wandb and wandb is not None and wandb.run is not None:
            self.exp_dir.mkdir(parents=True, exist_ok=True)
            (self.exp_dir / "wandb_run_id.txt").write_text(wandb.run.id)
        ckpt.save_worker_state(ckpt_dir, train_reader=self.train_reader)
        # every rank's shard file is on disk before any rank passes the barrier and before rank 0 copies the directory
        ckpt.finish_pending_shard_writes()
        if dist.is_available() and dist.is_initialized():
            dist.barrier()
        if self.master:
            ckpt.rsync_if_slurm(ckpt_dir)
            print(f"[Checkpoint] END   {label} iter={self.curr_iter} -> {ckpt_dir}")

    def maybe_checkpoint(self):
        cfg, it = self.cfg, self.curr_iter
        if cfg.permanent_ckpt_interval > 0 and it % cfg.permanent_ckpt_interval == 0:
            self._write_checkpoint(self.exp_dir / "ckpts" / str(it), "permanent")
        if cfg.latest_ckpt_interval > 0 and (it % cfg.latest_ckpt_interval == 0 or it == cfg.iterations):
            self._write_checkpoint(self.exp_dir / "ckpts" / "latest", "latest   ")

    # ---- evaluation ---------------------------------------------------------------------------------------
    def eval_and_log(self, tokens, epoch, full_eval=False):
        cfg, it = self.cfg, self.curr_iter
        if not (self.all_ranks_ckpt or self.collective_forward) and not self.master:
            return
        self.model.eval()
        if cfg.opt in ("sf-sgd", "sf-adamw"):
            self.opt.eval()
        n = self.val_reader.num_batches() if (it == cfg.iterations or full_eval) else cfg.eval_batches
        self.val_reader.set_step(0)
        acc, loss, pp, aux, router = evaluate(self.run_model, self.val_reader, cfg.device, max_num_batches=n,
                                              ctx=self.type_ctx, moe=cfg.moe,
                                              get_router_logits=cfg.moe and cfg.plot_router_logits, cfg=cfg)
        if self.master:
            print(f">Eval: Iter={it} ({epoch:0.3f} epochs) val_loss={loss:.3f} val_pp={pp:.3f} val_acc={acc:3f}")
            self.stats["val_loss"].append(loss)
            self.stats["val_pp"].append(pp)
            self.stats["val_acc"].append(acc)
            prefix = "final-val" if (it == cfg.iterations or full_eval) else "val"
            logs = {"tokens": tokens, "iter": it, f"{prefix}/loss": loss, f"{prefix}/perplexity": pp,
                    f"{prefix}/acc": acc, **aux}
            if cfg.wandb and wandb is not None and cfg.moe and cfg.plot_router_logits:
                from ..logging.routing import visualize_routing

                logs.update(visualize_routing(router, cfg))
            self.sink.log(logs, step=it)
            if cfg.wandb and wandb is not None:
                if cfg.eval_seq_prefix != "none" and (it % (cfg.eval_interval * 5) == 0 or it == cfg.iterations):
                    table = wandb.Table(columns=["itr", "val-pp", "text"])
                    text = self.backend.get_raw_model(self.model).generate_from_string(
                        cfg.eval_seq_prefix, max_new_tokens=40, temperature=0.9, top_k=None)
                    table.add_data(it, pp, text)
                    wandb.log({f"generated-text-{wandb.run.name}": copy.copy(table)}, step=it)
        self.model.train()

    # ---- one optimizer step ----------------------------------------------------------------------------------
    def train_step(self):
        cfg, model, opt = self.cfg, self.run_model, self.opt
        outputs, loss, x, y = None, None, None, None
        if self.engine is not None:
            # auxiliary values that do not enter the loss are only computed on iterations whose outputs are logged
            self.engine.report_aux = bool(cfg.log_interval) and (self.curr_iter + 1) % cfg.log_interval == 0
        for micro in range(cfg.acc_steps):
            with nvtx_range("data", cfg):
                x, y = self.stager.next_batch()
            with nvtx_range("forward", cfg), self.type_ctx, \
                    self.backend.get_context_for_microstep_forward(model=model, microstep_idx=micro,
                                                                   gradient_accumulation_steps=cfg.acc_steps):
                outputs = model(x, targets=y, moe=cfg.moe)
            loss = outputs["loss"] / cfg.acc_steps
            with nvtx_range("backward", cfg):
                loss.backward()
            self.substep += 1
        if cfg.grad_clip != 0.0:
            raw = self.backend.get_raw_model(self.model)
            gn = self.backend.clip_grad_norm_(raw.parameters(), cfg.grad_clip)
            self.grad_norms.append(gn)  # kept on the device; read only when logging
        if hasattr(opt, "want_diagnostics"):
            # the engine's fused optimizer reports the `optimizer/*` schedule metrics only when asked: ask on the
            # steps whose iteration will be logged
            opt.want_diagnostics = bool(cfg.log_interval) and (self.curr_iter + 1) % cfg.log_interval == 0
        with nvtx_range("optimizer", cfg):
            if self.engine is not None:
                self.engine.finish_grad_sync()    # (a per-tensor optimizer reads the gradient buffers directly)
            if cfg.opt in ("sf-sgd", "sf-adamw"):
                opt.train()
            if cfg.opt == "sophiag":
                opt.step(bs=cfg.sophia_bs * cfg.sequence_length)
            else:
                opt.step()
            if cfg.scheduler != "none" and self.scheduler is not None:
                self.scheduler.step()
            self._post_step_hooks(x, y)
        return outputs, loss

    def _post_step_hooks(self, x, y):
        cfg, opt = self.cfg, self.opt
        external_opt_on_engine = self.engine is not None and not getattr(self.backend, "engine_optimizer", False)
        if external_opt_on_engine:
            self.engine.refresh_from_master()
        if cfg.opt == "sophiag":
            opt.zero_grad(set_to_none=True)
            f = cfg.precondition_frequency
            if self.curr_iter % f == f - 1:
                if self.engine is not None and self.engine.sharded:
                    # no rank holds the module's parameters: the engine draws the labels chunk by chunk itself
                    self.engine.sync_on_backward = True
                    out = self.engine.forward(x, None, sample_targets=True)
                    (out["loss"] / cfg.acc_steps).backward()
                    self.engine.sync_on_backward = None
                else:
                    if self.engine is not None:
                        self.engine.enabled = False
                    out = self.run_model(x, targets=y, get_logits=True)
                    if self.engine is not None:
                        self.engine.enabled = True
                    logits = out["logits"]
                    y_s = torch.distributions.Categorical(logits=logits).sample()
                    l = torch.nn.functional.cross_entropy(logits.view(-1, logits.size(-1)), y_s.view(-1), ignore_index=-1)
                    (l / cfg.acc_steps).backward()
                opt.update_hessian()
                opt.zero_grad(set_to_none=True)
                self.model.zero_grad()
        elif cfg.opt == "mars":
            opt.zero_grad(set_to_none=True)
            opt.update_last_grad()
        if self.engine is not None and cfg.opt in ("sophiag", "mars"):
            # their branches above drop the gradients the way the reference does (`set_to_none`): restart the engine's
            # micro-step count and point the parameters' `.grad` back at the engine's gradient buffers
            self.engine.zero_grad()
        elif cfg.opt in ("sophiag", "mars"):
            pass
        elif self.engine is not None:
            self.engine.zero_grad()  # gradient buffers are overwritten by the next first micro-step
        else:
            opt.zero_grad(set_to_none=True)

    # ---- logging ---------------------------------------------------------------------------------------------
    def log_train(self, outputs, loss, dt, tokens, epoch):
        cfg, opt = self.cfg, self.opt
        train_loss = loss.detach().float().item() * cfg.acc_steps
        self.stats["train_loss"].append(train_loss)
        lrs = [g["lr"] for g in opt.param_groups]
        print(f"Train: Iter={self.curr_iter} ({epoch:0.3f} epochs) train_loss={train_loss:.3f} "
              f"iter_dt={dt:.2e}s lr={lrs[0]:.2e}")
        from ..logging.schedules import log_optimizer_schedules, log_prodigy_lr

        if cfg.opt == "prodigy":
            eff = log_prodigy_lr(opt)
            print(f"effective_lr={eff[0]:.2e}")
        if self.master:
            gns = [float(g) for g in self.grad_norms]
            logs = {"tokens": tokens, "iter": self.curr_iter, "train/loss": train_loss,
                    "train/perplexity": 2.71828 ** train_loss, "lr": lrs[0], "iter_dt": dt,
                    "max_grad_norm": max(gns) if gns else 0, "mean_grad_norm": sum(gns) / len(gns) if gns else 0,
                    **{f"train/{k}": float(v) for k, v in outputs["aux_losses"].items()}}
            if cfg.opt == "prodigy":
                logs["effective_lr"] = eff[0]
            logs.update(log_optimizer_schedules(opt, cfg.opt) or {})
            if cfg.log_parameter_norms:
                from ..logging.schedules import get_parameter_norms

                logs["model_norm"] = get_parameter_norms(self.backend.get_raw_model(self.model), order=cfg.norm_order)
            self.sink.log(logs, step=self.curr_iter)
        self.grad_norms = []

    # ---- main loop ---------------------------------------------------------------------------------------------
    def run(self):
        cfg = self.cfg
        self.setup()
        ws = self.backend.get_world_size()
        while self.curr_iter <= cfg.iterations:
            self.maybe_checkpoint()
            tokens = ws * self.substep * cfg.sequence_length * cfg.batch_size
            epoch = tokens / self.train_reader.num_tokens
            is_eval = (self.curr_iter % cfg.eval_interval == 0 or self.curr_iter == cfg.iterations
                       or self.curr_iter in cfg.full_eval_at)
            if is_eval:
                with self._phase("eval"):
                    self.eval_and_log(tokens, epoch, full_eval=self.curr_iter in cfg.full_eval_at)
                if self.tau_stats is not None and self.tau_stats.should_collect(self.curr_iter, is_eval):
                    self.tau_stats.collect(self.opt, self.curr_iter)
            if cfg.iterations_to_run is not None and self.iters_in_run >= cfg.iterations_to_run:
                self._write_checkpoint(self.exp_dir / "ckpts" / "latest",
                                       f"latest (iterations_to_run reached) iterations_in_run={self.iters_in_run}")
                if cfg.permanent_ckpt_interval > 0 and self.curr_iter % cfg.permanent_ckpt_interval == 0:
                    self._write_checkpoint(self.exp_dir / "ckpts" / str(self.curr_iter), "permanent")
                break
            if self.curr_iter == cfg.iterations:
                break
            if self._exit_at is not None and self.curr_iter == self._exit_at[0]:
                print(f"[Fault] leaving at iteration {self.curr_iter} (ADANA_FAULT_EXIT)", flush=True)
                if self.cuda:
                    torch.cuda.synchronize()
                os._exit(self._exit_at[1])
            if self.watchdog is not None:
                self.watchdog.beat(self.curr_iter)
                self.watchdog.raise_if_failed()
            t0 = time.perf_counter_ns()
            self.timer.start()
            outputs, loss = self.train_step()
            dt_dev = self.timer.stop()
            dt = dt_dev if dt_dev is not None else (time.perf_counter_ns() - t0) / 1e9
            self.curr_iter += 1
            self.iters_in_run += 1
            if self.curr_iter == 1 and self.master and self.cuda:
                print(f"[Memory] GPU 0: peak_allocated={torch.cuda.max_memory_allocated() / 1024 ** 3:.2f} GiB, "
                      f"peak_reserved={torch.cuda.max_memory_reserved() / 1024 ** 3:.2f} GiB")
            if cfg.log_interval and self.curr_iter % cfg.log_interval == 0:
                self.check_device_status()
                if self.master:
                    self.log_train(outputs, loss, dt, tokens, epoch)
        self.check_device_status()
        if self.watchdog is not None:
            self.watchdog.stop()
        ckpt.finish_pending_writes()
        return self.stats


def train(model, opt, datareaders, scheduler, exp_dir, distributed_backend, cfg):
    return Trainer(model, opt, datareaders, scheduler, exp_dir, distributed_backend, cfg).run()
