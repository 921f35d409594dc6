"""Multi-process CPU tests (gloo, world size 2): data-parallel, sharded-optimizer, expert-parallel and pipeline
plumbing must reproduce the single-process result."""

import pytest
import torch

from gpt_moe_b200.config import get_preset

from dist_helpers import run_ranks


def _config(**model_kw):
    gc, tc = get_preset("tiny_cpu")
    gc.n_layers, gc.hidden_size, gc.attn_dim, gc.n_heads, gc.n_kv_heads = 2, 64, 64, 2, 2
    gc.mlp_hidden_dim, gc.vocab_size, gc.weighted_main_path_init = 64, 512, 0.5
    for k, v in model_kw.items():
        setattr(gc, k, v)
    tc.gpu_batch_size_train = tc.gpu_batch_size_val = 2
    tc.seq_len_train = tc.seq_len_val = 32
    tc.kernel_warmup_train_steps = 0
    tc.grad_bucket_mb = 1
    return gc, tc


def _batches(steps, rows, seq, vocab):
    gen = torch.Generator().manual_seed(123)
    return [torch.randint(0, vocab, (rows, seq + 1), generator=gen) for _ in range(steps)]


def _train(rank, world, model_kw, train_kw, steps):
    from gpt_moe_b200.runtime.trainer import Trainer
    gc, tc = _config(**model_kw)
    for k, v in train_kw.items():
        setattr(tc, k, v)
    trainer = Trainer(gc, tc, device_type="cpu", quiet=True)
    rows = tc.gpu_batch_size_train
    losses = []
    for ids in _batches(steps, rows * world, tc.seq_len_train, gc.vocab_size):
        mine = ids[rank * rows: (rank + 1) * rows]
        losses.append(trainer.train_step([(mine[:, :-1].contiguous(), mine[:, 1:].contiguous(), None)])["token_loss"])
    from gpt_moe_b200.checkpointing.checkpoint import gather_full_state_dict
    state = gather_full_state_dict(trainer.raw_gpt_model, trainer.ep_group)
    opt = trainer.engine.full_optimizer_state_dicts() if hasattr(trainer.engine, "full_optimizer_state_dicts") else None
    return {"losses": losses, "state": state, "muon_state_count": None if opt is None else len(opt["muon"]["state"])}


def _single(model_kw, train_kw, steps, world):
    """Single-process oracle: same global batch, gradient = mean over the rank shards (equal token counts)."""
    from gpt_moe_b200.models.gpt import GPT
    gc, tc = _config(**model_kw)
    for k, v in train_kw.items():
        if k not in ("expert_parallel_size", "parallel_mode"):
            setattr(tc, k, v)
    tc.resolve(1)
    torch.manual_seed(tc.base_seed)
    model = GPT(gc, tc)
    opts = model.configure_optimizers(tc.adamw_max_lr, tc.adamw_betas, tc.adamw_eps, tc.adamw_weight_decay, "cpu")
    rows = tc.gpu_batch_size_train
    losses, tokens = [], 0
    for ids in _batches(steps, rows * world, tc.seq_len_train, gc.vocab_size):
        step_losses = []
        for r in range(world):
            mine = ids[r * rows: (r + 1) * rows]
            loss, token_loss, _ = model(mine[:, :-1], mine[:, 1:])
            (loss / world).backward()
            step_losses.append(token_loss.item())
        lr = tc.lr_schedule[0]["fn"](tokens, **tc.lr_schedule[0]["kwargs"])
        for g in opts["adamw"].param_groups:
            g["lr"] = lr
        for g in opts["muon"].param_groups:
            g["lr"] = lr * tc.muon_lr_scale
        for o in opts.values():
            o.step()
            o.zero_grad()
        tokens += rows * tc.seq_len_train * world
        losses.append(sum(step_losses) / world)
    return losses, model.state_dict()


def _compare(result, oracle_losses, oracle_state, atol=2e-4):
    assert result["losses"] == pytest.approx(oracle_losses if not isinstance(oracle_losses[0], list) else oracle_losses, abs=1e-3)
    for name, want in oracle_state.items():
        got = result["state"][name]
        assert torch.allclose(got, want, atol=atol, rtol=1e-3), (name, (got - want).abs().max().item())


@pytest.mark.parametrize("shard", [False, True])
def test_data_parallel_matches_single_process(tmp_path, shard):
    results = run_ranks(_train, 2, tmp_path, {}, {"shard_muon": shard}, 3)
    # each rank logs its own shard's loss; their mean is the global loss
    mean_losses = [(a + b) / 2 for a, b in zip(results[0]["losses"], results[1]["losses"])]
    oracle_losses, oracle_state = _single({}, {}, 3, 2)
    assert mean_losses == pytest.approx(oracle_losses, abs=1e-3)
    for r in results:
        for name, want in oracle_state.items():
            assert torch.allclose(r["state"][name], want, atol=2e-4, rtol=1e-3), name
    if shard:
        assert results[0]["muon_state_count"] == 26      # gathered optimizer state covers every Muon matrix


def test_expert_parallel_matches_replicated(tmp_path):
    results = run_ranks(_train, 2, tmp_path, {"moe_top_k": 2}, {"expert_parallel_size": 2, "shard_muon": False}, 2)
    oracle_losses, oracle_state = _single({"moe_top_k": 2}, {}, 2, 2)
    mean_losses = [(a + b) / 2 for a, b in zip(results[0]["losses"], results[1]["losses"])]
    assert mean_losses == pytest.approx(oracle_losses, abs=1e-3)
    for r in results:
        assert set(r["state"]) == set(oracle_state)          # experts gathered back under their global indices
        for name, want in oracle_state.items():
            assert torch.allclose(r["state"][name], want, atol=3e-4, rtol=1e-3), name


def _pipeline(rank, world, steps):
    from gpt_moe_b200.runtime.trainer import Trainer
    gc, tc = _config()
    tc.parallel_mode = "pp"
    tc.total_tokens_per_step_train = 2 * tc.gpu_batch_size_train * tc.seq_len_train     # two micro-batches per step
    trainer = Trainer(gc, tc, device_type="cpu", quiet=True)
    rows = tc.gpu_batch_size_train
    out = []
    for ids in _batches(steps, rows * 2, tc.seq_len_train, gc.vocab_size):
        batches = []
        for m in range(2):
            mine = ids[m * rows: (m + 1) * rows]
            batches.append((mine[:, :-1].contiguous() if rank == 0 else None, mine[:, 1:].contiguous(), None))
        trainer.engine.zero_grad()
        losses = trainer.pipeline_runtime.train_step(batches)
        torch.distributed.all_reduce(losses)
        trainer.engine.step()
        out.append(losses[1].item())
    return {"losses": out, "state": dict(trainer.raw_gpt_model.state_dict())}


def test_two_stage_pipeline_matches_single_process(tmp_path):
    results = run_ranks(_pipeline, 2, tmp_path, 2)
    gc, tc = _config()
    tc.resolve(1)
    from gpt_moe_b200.models.gpt import GPT
    torch.manual_seed(tc.base_seed)
    model = GPT(gc, tc)
    opts = model.configure_optimizers(tc.adamw_max_lr, tc.adamw_betas, tc.adamw_eps, tc.adamw_weight_decay, "cpu")
    rows = tc.gpu_batch_size_train
    losses = []
    for ids in _batches(2, rows * 2, tc.seq_len_train, gc.vocab_size):
        acc = 0.0
        for m in range(2):
            mine = ids[m * rows: (m + 1) * rows]
            loss, token_loss, _ = model(mine[:, :-1], mine[:, 1:])
            (loss / 2).backward()
            acc += token_loss.item() / 2
        for o in opts.values():
            o.step()
            o.zero_grad()
        losses.append(acc)
    assert results[1]["losses"] == pytest.approx(losses, abs=1e-3)
    full = model.state_dict()
    for name, got in results[0]["state"].items():
        assert torch.allclose(got, full[name], atol=2e-4, rtol=1e-3), name
    for name, got in results[1]["state"].items():
        if name.startswith("transformer.h."):
            parts = name.split(".")
            parts[2] = str(int(parts[2]) + 1)
            name = ".".join(parts)
        assert torch.allclose(got, full[name], atol=2e-4, rtol=1e-3), name


def test_expert_replicas_reduce_only_among_themselves(tmp_path):
    """World 4 with expert_parallel_size 2: ranks 0/2 and 1/3 hold the same experts.  Expert gradients are summed over those
    replica pairs only (and nothing else's), so the run reproduces the single-process result and the replicas stay equal."""
    results = run_ranks(_train, 4, tmp_path, {"moe_top_k": 2}, {"expert_parallel_size": 2, "shard_muon": True}, 2, join_timeout=480)
    oracle_losses, oracle_state = _single({"moe_top_k": 2}, {}, 2, 4)
    mean_losses = [sum(r["losses"][i] for r in results) / 4 for i in range(2)]
    assert mean_losses == pytest.approx(oracle_losses, abs=1e-3)
    for r in results:
        assert set(r["state"]) == set(oracle_state)
        for name, want in oracle_state.items():
            assert torch.allclose(r["state"][name], want, atol=3e-4, rtol=1e-3), name
        assert r["muon_state_count"] == 26          # every Muon matrix of the unsharded model exactly once


def _train_save_resume(rank, world, train_kw, ckpt_dir, resume):
    """Three steps and a save; or (resume) a fresh trainer from that save, one more step and a second save."""
    import os
    from gpt_moe_b200.runtime.trainer import Trainer
    gc, tc = _config(moe_top_k=2)
    for k, v in train_kw.items():
        setattr(tc, k, v)
    tc.checkpoint_dir = os.path.join(ckpt_dir, "resumed" if resume else "first")
    if resume:
        first = os.path.join(ckpt_dir, "first")
        weights = [f for f in os.listdir(first) if f.startswith("model_step_0000002")][0]
        tc.resume_from_checkpoint = True
        tc.resume_checkpoint_path = os.path.join(first, weights)
        tc.resume_state_dict_path = os.path.join(first, "training_state_step_0000002.pt")
    trainer = Trainer(gc, tc, device_type="cpu", quiet=True)
    rows = tc.gpu_batch_size_train
    batches = _batches(4, rows * world, tc.seq_len_train, gc.vocab_size)
    steps = range(3, 4) if resume else range(4)
    for i in steps:
        mine = batches[i][rank * rows: (rank + 1) * rows]
        trainer.train_step([(mine[:, :-1].contiguous(), mine[:, 1:].contiguous(), None)])
        if not resume and i == 2:
            trainer.save(2, 0.0, None)
    trainer.save(3, 0.0, None)
    return {"dir": tc.checkpoint_dir}


@pytest.mark.parametrize("ep", [1, 2])
def test_sharded_checkpoint_resume_saves_the_same_state_as_an_uninterrupted_run(tmp_path, ep):
    """Two ranks with the sharded optimizer (and with expert parallelism): save after step 2, resume in fresh processes, take
    step 3 and save again.  Weights and every optimizer entry of that second save equal the uninterrupted run's save after
    step 3 — stale momentum of non-owned matrices or expert state keyed by a local index would show up here."""
    import os
    from safetensors.torch import load_file
    kw = {"expert_parallel_size": ep, "shard_muon": True}
    work, ckpt_dir = tmp_path / "work", tmp_path / "ckpt"
    for d in (work / "a", work / "b", ckpt_dir):
        os.makedirs(d)
    run_ranks(_train_save_resume, 2, work / "a", kw, str(ckpt_dir), False)
    run_ranks(_train_save_resume, 2, work / "b", kw, str(ckpt_dir), True)

    def load(sub):
        folder = ckpt_dir / sub
        weights = [f for f in os.listdir(folder) if f.startswith("model_step_0000003")][0]
        return load_file(str(folder / weights)), torch.load(str(folder / "training_state_step_0000003.pt"), weights_only=False)

    w_first, s_first = load("first")
    w_resumed, s_resumed = load("resumed")
    assert set(w_first) == set(w_resumed)
    for name in w_first:
        assert torch.allclose(w_first[name], w_resumed[name], atol=1e-6), name
    for opt in ("muon", "adamw"):
        a, b = s_first["optimizer_state_dicts"][opt], s_resumed["optimizer_state_dicts"][opt]
        assert a["param_groups"][0]["params"] == b["param_groups"][0]["params"]
        assert set(a["state"]) == set(b["state"]) and len(a["state"]) > 0
        for key in a["state"]:
            for field, value in a["state"][key].items():
                other = b["state"][key][field]
                if isinstance(value, torch.Tensor):
                    assert torch.allclose(value.float(), other.float(), atol=1e-6), (opt, key, field)
    assert len(s_first["optimizer_state_dicts"]["muon"]["state"]) == 26      # unsharded layout: every Muon matrix once


def _pipeline_warmup(rank, world):
    from gpt_moe_b200.runtime.trainer import Trainer
    from gpt_moe_b200.runtime.warmup import kernel_warmup
    gc, tc = _config()
    tc.parallel_mode = "pp"
    tc.total_tokens_per_step_train = 2 * tc.gpu_batch_size_train * tc.seq_len_train
    trainer = Trainer(gc, tc, device_type="cpu", quiet=True)
    before = {n: p.detach().clone() for n, p in trainer.raw_gpt_model.named_parameters()}
    rng = torch.get_rng_state()
    elapsed = kernel_warmup(trainer.run, num_train_steps=1)
    same = all(torch.equal(p.detach(), before[n]) for n, p in trainer.raw_gpt_model.named_parameters())
    empty_state = all(not entry for o in trainer.optimizers.values() for entry in o.state_dict()["state"].values())
    return {"elapsed": elapsed, "same": same, "empty_state": empty_state, "rng": torch.equal(rng, torch.get_rng_state()),
            "tokens": trainer.train_tokens_processed}


def test_pipeline_warmup_runs_both_stages_and_restores(tmp_path):
    """The warm-up in pipeline mode takes real 1F1B steps and a forward-only pass on both stages, then puts weights,
    optimizer state, RNG and counters back exactly."""
    results = run_ranks(_pipeline_warmup, 2, tmp_path)
    for r in results:
        assert r["elapsed"] > 0.0 and r["same"] and r["empty_state"] and r["rng"] and r["tokens"] == 0
