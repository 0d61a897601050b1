"""Drive the unmodified reference (installed under ``baseline/_ref``) for the benchmarks' ``--impl reference`` arms.

``run_train_steps`` repeats the body of the reference's own training loop (``nmoe/train.py:88-109``: ``update_lr`` ->
``loader.next()`` -> ``model(inputs)`` -> masked cross-entropy -> ``zero_grad`` -> ``backward`` -> ``opt.step``) on its
own objects: ``nmoe.config.Config``, ``nmoe.model.Transformer``, ``nmoe.data.loader.build_loader`` (its ``data_path``
fast path over synthetic ``.npy`` shards), ``nmoe.opt.build_optimizer`` / ``update_lr`` / ``step``.  The loop is
restated here only because the stock ``train()`` offers no place to put CUDA events around exactly K steps, and because
``nmoe/metrics.py`` imports duckdb, which this image does not have; logging, checkpointing and evaluation are left out
of the timed loop, which can only flatter the reference.  None of this repository's kernels, models or engine runs.

``moe_layer`` builds the reference's ``Rdep`` and calls ``moe_bf16`` / ``moe_blockscaled`` as its ``MoE.forward`` does
(``nmoe/model.py:113-138``), for the layer- and RDEP-level micro-benchmarks.
"""
from __future__ import annotations

import os
import shutil
import tempfile
import time

from . import ref_env


def _max_over_ranks(ms: float, world: int, device) -> float:
    import torch
    import torch.distributed as dist
    if world == 1:
        return ms
    t = torch.tensor([ms], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _barrier(world: int) -> None:
    import torch
    import torch.distributed as dist
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def write_synthetic_shards(path: str, n_tokens: int, vocab: int, seed: int = 1234) -> None:
    """One uint32 ``.npy`` shard of uniform-random token ids (the format nmoe/data/dataset.py:27-33 memory-maps)."""
    import numpy as np
    os.makedirs(path, exist_ok=True)
    rng = np.random.default_rng(seed)
    arr = rng.integers(0, vocab - 1, size=int(n_tokens), dtype=np.uint32)
    np.save(os.path.join(path, "synthetic_000.npy"), arr)


def run_train_steps(model_fields: dict, *, micro_batch: int, seq_len: int, steps: int, warmup: int, dtype: str,
                    e2e: bool = True, before_timed=None, after_timed=None) -> dict:
    """Train the reference model for `warmup` untimed and `steps` timed steps; returns timings (max over ranks).

    `model_fields` are keyword arguments of the reference's Config (architecture and optimiser settings)."""
    os.environ.setdefault("NMOE_TIMERS", "0")
    ref_env.activate()
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F
    from nmoe import runtime as ref_runtime
    from nmoe.config import Config as RefConfig

    rank, world = ref_runtime.init(42)
    device = torch.device("cuda", torch.cuda.current_device())
    if dtype != "bf16" and not ref_env.blockscaled_available():
        raise ref_env.ReferenceUnavailable(f"reference dtype={dtype} needs nmoe/blockscaled/grouped.py, which is not in "
                                           "this snapshot")
    total_steps = warmup + steps * (2 if e2e else 1) + 2
    batch = micro_batch * world
    work = None
    box = [None]
    if rank == 0:
        work = tempfile.mkdtemp(prefix="nmoe_ref_arm_")
        need = total_steps * batch * (seq_len + 1)
        write_synthetic_shards(os.path.join(work, "data"), min(need, 48 << 20), model_fields["vocab_size"])
        box[0] = work
    if world > 1:
        dist.broadcast_object_list(box, src=0)
    work = box[0]
    try:
        cfg = RefConfig(**model_fields, dtype=dtype, batch_size=batch, seq_len=seq_len, steps=total_steps, seed=42,
                        data_path=os.path.join(work, "data"), checkpoint_dir=os.path.join(work, "ckpt"),
                        metrics_dir=os.path.join(work, "metrics"), experiments_db=os.path.join(work, "exp.db"),
                        resume=False)
        from nmoe.data.loader import build_loader
        from nmoe.model import Transformer
        from nmoe.opt import build_optimizer, step as opt_step, update_lr

        quiet = (lambda *a, **k: None)
        loader, _plan = build_loader(cfg, rank, world, print_fn=quiet)
        with torch.device(device):          # parameters are created on the GPU instead of being copied from the host
            model = Transformer(cfg)
        model = model.cuda()
        model.init_weights()
        model.train()
        optimizer, dense_groups = build_optimizer(model, cfg)
        zero2_state: dict = {}
        tokens_seen = 0
        step_num = 0

        def one_step():
            nonlocal tokens_seen, step_num
            update_lr(optimizer, dense_groups, step_num, tokens_seen, cfg)
            inputs, targets = loader.next()
            logits = model(inputs)
            loss_unreduced = F.cross_entropy(logits.reshape(-1, cfg.vocab_size), targets.reshape(-1), reduction="none")
            mask = (targets != cfg.eos_token_id).reshape(-1).float()
            loss = (loss_unreduced * mask).sum() / mask.sum().clamp(min=1.0)
            model.zero_grad(set_to_none=True)
            loss.backward()
            opt_step(model, optimizer, dense_groups, zero2_state, cfg, world)
            tokens_seen += cfg.batch_size * cfg.seq_len
            step_num += 1
            return loss.detach()

        for _ in range(warmup):
            one_step()
        _barrier(world)
        if before_timed is not None:
            before_timed()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        _barrier(world)
        ev0.record()
        for _ in range(steps):
            loss = one_step()
        ev1.record()
        _barrier(world)
        if after_timed is not None:
            after_timed()
        ms = _max_over_ranks(ev0.elapsed_time(ev1), world, device)
        final_loss = float(loss.item())
        out = {"ms": ms, "final_loss": final_loss, "world": world, "rank": rank,
               "peak_mem_gib": torch.cuda.max_memory_allocated() / 2 ** 30}
        if e2e:
            _barrier(world)
            t0 = time.perf_counter()
            ev0.record()
            for _ in range(steps):
                _ = one_step().item()
            ev1.record()
            _barrier(world)
            wall = (time.perf_counter() - t0) * 1e3
            out["e2e_ms"] = _max_over_ranks(max(ev0.elapsed_time(ev1), wall), world, device)
            out["h2d_bytes_per_step"] = int(batch * (seq_len + 1) * 8)
            out["d2h_bytes_per_step"] = int(4 * world)
        try:
            loader.close()
        except Exception:
            pass
        _barrier(world)
        return out
    finally:
        if rank == 0 and work:
            shutil.rmtree(work, ignore_errors=True)


class RefMoELayer:
    """The reference's routed-expert layer on its stock objects: `Rdep` + `moe_bf16` / `moe_blockscaled`.

    Weights follow nmoe/model.py:93-95 (`W1`, `W3` [E_local, H, Dff]; `W2` [E_local, Dff, H])."""

    def __init__(self, hidden: int, dff: int, n_experts: int, topk: int, tokens_per_rank: int, profile: str = "bf16",
                 seed: int = 0):
        ref_env.activate()
        import torch
        import torch.distributed as dist
        from nmoe.rdep import Rdep
        self.torch = torch
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        if n_experts % self.world:
            raise ValueError("experts must divide over ranks")
        if profile != "bf16" and not ref_env.blockscaled_available():
            raise ref_env.ReferenceUnavailable("blockscaled profile needs nmoe/blockscaled/grouped.py")
        self.n_local = n_experts // self.world
        self.profile = profile
        self.rdep = Rdep(hidden, self.n_local, topk, profile=profile,
                         capacity=int(tokens_per_rank) * topk * self.world)
        g = torch.Generator(device="cuda").manual_seed(seed + 17 * self.rank)
        mk = lambda *s: (torch.randn(*s, device="cuda", generator=g, dtype=torch.float32) * 0.02).bfloat16().requires_grad_(True)
        self.W1, self.W3, self.W2 = mk(self.n_local, hidden, dff), mk(self.n_local, hidden, dff), mk(self.n_local, dff, hidden)
        self.cache = None
        if profile != "bf16":
            from nmoe.blockscaled.grouped import quantize_weights
            self.cache = quantize_weights(self.W1, self.W3, self.W2, profile=profile)

    def forward(self, x, eid, gates):
        if self.cache is not None:
            return self.rdep.moe_blockscaled(x, eid, gates, self.W1, self.W3, self.W2, self.cache)
        return self.rdep.moe_bf16(x, eid, gates, self.W1, self.W3, self.W2)
