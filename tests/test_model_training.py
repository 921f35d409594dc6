import copy
import os

import numpy as np
import pytest
import torch

from gpt_moe_b200.config import build_resume_config, get_preset
from gpt_moe_b200.models.gpt import GPT


def tiny(**model_kw):
    gc, tc = get_preset("tiny_cpu")
    for k, v in model_kw.items():
        setattr(gc, k, v)
    tc.resolve(1)
    return gc, tc


def test_state_dict_layout_matches_reference_names():
    gc, tc = tiny()
    keys = set(GPT(gc, tc).state_dict().keys())
    expected = {"transformer.wte.weight", "transformer.ln_f.weight", "lm_head.weight"}
    for i in range(2):
        p = f"transformer.h.{i}."
        expected |= {p + "ln_1.weight", p + "ln_2.weight", p + "attn_main_scale", p + "mlp_main_scale",
                     p + "attn.q_scale", p + "attn.k_scale", p + "mlp.router.weight"}
        expected |= {p + f"attn.{n}.weight" for n in ("q_proj", "k_proj", "v_proj", "out_proj")}
        expected |= {p + f"mlp.experts.{e}.{n}.weight" for e in range(4) for n in ("up_proj", "down_proj")}
    assert keys == expected       # no rotary tables, no window buffer, no caches
    m = GPT(gc, tc)
    assert m.transformer.h[0].attn.q_scale.shape == (1, 4, 1, 1)
    assert m.transformer.h[0].mlp.experts["0"].up_proj.weight.shape == (1024, 128)     # SwiGLU: [2*hidden, d], gate first


def test_optimizer_split_follows_reference_rules():
    gc, tc = tiny()
    groups = GPT(gc, tc).optimizer_param_groups()
    muon = {n for n, _ in groups["muon"]}
    assert "transformer.h.0.mlp.router.weight" in muon and "transformer.h.1.attn.out_proj.weight" in muon
    assert not any(t in n for n in muon for t in ("wte", "lm_head"))
    decay = {n for n, _ in groups["adamw_decay"]}
    # the rule is dimensionality, as in the reference: the (1, H, 1, 1) QK scales are 4-D and therefore decayed
    assert {"transformer.wte.weight", "lm_head.weight", "transformer.h.0.attn.q_scale"} <= decay
    assert all(p.dim() >= 2 for _, p in groups["adamw_decay"])
    assert all(p.dim() < 2 for _, p in groups["adamw_nodecay"])


def test_variants_run_forward_backward():
    torch.manual_seed(0)
    ids = torch.randint(0, 50304, (2, 65))
    x, y = ids[:, :-1], ids[:, 1:]
    variants = [
        dict(n_kv_heads=2), dict(n_kv_heads=1), dict(use_moe=False, activation="gelu"), dict(activation="relu2", moe_top_k=2),
        dict(pos_encoding_type="nope"), dict(pos_encoding_type="absolute"), dict(norm_type="layer"),
        dict(use_weighted_residual_path=True), dict(use_weighted_residual_path=False, use_weighted_main_path=False),
        dict(use_qk_norm=False), dict(qk_norm_type="l2"), dict(use_attn_logit_softcapping=True, tanh_backend="rational"),
        dict(use_doc_masking=True), dict(full_attention_layers=[1], global_attn_dim=64, global_n_kv_heads=2),
        dict(use_tied_embeddings=True), dict(moe_shared_expert_hidden_dim=64), dict(moe_full_softmax_gating=True, moe_top_k=2),
        dict(use_mla=True, mla_kv_rank=32, mla_qk_content_dim=16, mla_qk_rope_dim=16, mla_value_dim=32),
        dict(use_mla=True, mla_q_rank=24, mla_kv_rank=32, mla_qk_content_dim=16, mla_qk_rope_dim=16, mla_value_dim=32, n_kv_heads=2),
    ]
    for kw in variants:
        gc, tc = tiny(**kw)
        model = GPT(gc, tc)
        docs = torch.zeros_like(x, dtype=torch.int32) if kw.get("use_doc_masking") else None
        loss, token_loss, balance = model(x, y, document_ids=docs)
        loss.backward()
        assert torch.isfinite(loss), kw
        model.eval()
        with torch.no_grad():
            assert model(x).shape == (2, 64, gc.vocab_size)
            assert model(x, y).dim() == 0


def test_sliding_window_changes_the_function_only_beyond_the_window():
    torch.manual_seed(1)
    gc, tc = tiny(weighted_main_path_init=1.0)
    model = GPT(gc, tc).eval()
    ids = torch.randint(0, 50304, (1, 64))
    with torch.no_grad():
        model.set_sliding_window(256)
        full = model(ids)
        model.set_sliding_window(8)
        local = model(ids)
    assert torch.allclose(full[:, :9], local[:, :9], atol=1e-5)      # positions 0..8 see the same W+1 = 9 keys
    assert not torch.allclose(full[:, 20:], local[:, 20:], atol=1e-5)


def test_mla_cached_decode_matches_full_forward():
    torch.manual_seed(2)
    gc, tc = tiny(use_mla=True, mla_kv_rank=32, mla_qk_content_dim=16, mla_qk_rope_dim=16, mla_value_dim=32, n_kv_heads=2)
    from gpt_moe_b200.models.attention import AttentionContext
    attn = GPT(gc, tc).transformer.h[0].attn.eval()
    x = torch.randn(2, 12, gc.hidden_size)
    with torch.no_grad():
        full = attn(x, AttentionContext(None, None, None))
        cache = attn.allocate_cache(2, 16, device="cpu", dtype=torch.float32)
        first = attn.forward_cached(x[:, :8], cache)
        rest = torch.cat([attn.forward_cached(x[:, i:i + 1], cache) for i in range(8, 12)], dim=1)
    assert torch.allclose(torch.cat((first, rest), dim=1), full, atol=1e-4)
    assert cache.length == 12 and cache.latent.shape == (2, 16, 32)


def test_ten_step_loss_curve_is_reproducible_and_decreases():
    """Tiny GPT-MoE on CPU, fp32: 2 layers, d_model 128, 4 heads x 32, 4 SwiGLU experts top-1, seq 256, micro-batch 4,
    uniform token ids from seed 0, Muon (Polar Express) + AdamW.  Residual gates start at 0.5 here so the blocks
    contribute from step 0 (the reference default of 0.0 makes every block a no-op at initialisation)."""
    def run():
        torch.manual_seed(0)
        gc, tc = tiny(weighted_main_path_init=0.5)
        model = GPT(gc, tc)
        opts = model.configure_optimizers(tc.adamw_max_lr, tc.adamw_betas, tc.adamw_eps, tc.adamw_weight_decay, "cpu")
        gen = torch.Generator().manual_seed(0)
        ids = torch.randint(0, 50304, (4, 257), generator=gen)     # one fixed batch: the curve must fall
        losses = []
        for _ in range(10):
            loss, _, _ = model(ids[:, :-1], ids[:, 1:])
            loss.backward()
            for o in opts.values():
                o.step()
                o.zero_grad()
            losses.append(loss.item())
        return losses
    a, b = run(), run()
    assert a == b
    assert a[-1] < a[0] - 1.0, a
    golden = os.path.join(os.path.dirname(__file__), "golden_tiny_loss_curve.json")
    import json
    if os.path.exists(golden):
        want = json.load(open(golden))
        assert np.allclose(a, want, rtol=2e-3), (a, want)


def test_checkpoint_roundtrip_and_resume_guard(tmp_path):
    from gpt_moe_b200.checkpointing import checkpoint as ckpt
    from safetensors.torch import load_file
    torch.manual_seed(3)
    gc, tc = tiny()
    model = GPT(gc, tc)
    opts = model.configure_optimizers(1e-3, (0.9, 0.95), 1e-8, 0.01, "cpu")
    ids = torch.randint(0, 50304, (2, 33))
    model(ids[:, :-1], ids[:, 1:])[0].backward()
    for o in opts.values():
        o.step()
    rc = build_resume_config(gc, tc)
    rng = [{"cpu": torch.get_rng_state(), "cuda": torch.empty(0, dtype=torch.uint8)}]
    path = ckpt.save_checkpoint(str(tmp_path), model, [], step=7, rng_states_by_rank=rng, val_loss=None, train_loss=3.14159,
                                train_tokens_processed=123, total_train_t=1.0, total_val_t=0.0, total_sample_t=0.0,
                                total_hellaswag_t=0.0, total_t=1.0, best_val_loss=float("inf"), epoch=0, current_shard_idx=0,
                                grad_accum_mini_steps_per_shard_counter=5, optimizers=opts, parallel_mode="ddp", world_size=1,
                                rank=0, resume_config=rc, schedule_state={"swa_schedule_idx": 0}, best_improvement_count=0,
                                allow_val=False)
    assert os.path.basename(path) == "model_step_0000007_val_na_train_3.1416.safetensors"
    state_path = os.path.join(str(tmp_path), "training_state_step_0000007.pt")
    ts = torch.load(state_path, weights_only=False)
    assert set(ts) == set(ckpt.TRAINING_STATE_KEYS) and ts["format_version"] == 2
    muon_state = ts["optimizer_state_dicts"]["muon"]["state"]
    assert all(set(s) == {"momentum_buffer"} for s in muon_state.values())
    adam_state = ts["optimizer_state_dicts"]["adamw"]["state"]
    assert all(set(s) == {"step", "exp_avg", "exp_avg_sq"} for s in adam_state.values())
    assert set(load_file(path)) == set(model.state_dict())

    tc.resume_from_checkpoint, tc.resume_checkpoint_path, tc.resume_state_dict_path = True, path, state_path
    loaded = ckpt.load_checkpoint(tc, gc, 0, 1, rc)
    assert loaded["start_step"] == 8 and loaded["grad_accum_mini_steps_per_shard_counter"] == 5
    for (n, a), (_, b) in zip(model.state_dict().items(), loaded["gpt_model"].state_dict().items()):
        assert torch.equal(a, b), n
    changed = copy.deepcopy(rc)
    changed["model"]["n_layers"] = 3
    with pytest.raises(ValueError, match="configuration differs"):
        ckpt.load_checkpoint(tc, gc, 0, 1, changed)
    with pytest.raises(ValueError, match="GPU count"):
        ckpt.load_checkpoint(tc, gc, 0, 2, rc)
    # rotation keeps the newest N steps
    for step in (8, 9, 10):
        open(os.path.join(str(tmp_path), f"model_step_{step:07d}_val_na_train_1.0000.safetensors"), "w").close()
        open(os.path.join(str(tmp_path), f"training_state_step_{step:07d}.pt"), "w").close()
    ckpt.keep_latest_checkpoints(str(tmp_path), 2, [])
    left = sorted(os.listdir(str(tmp_path)))
    assert all("0000009" in f or "0000010" in f for f in left) and len(left) == 4


def test_tied_embedding_checkpoint_loads_from_either_key(tmp_path):
    from gpt_moe_b200.checkpointing import checkpoint as ckpt
    gc, tc = tiny(use_tied_embeddings=True)
    model = GPT(gc, tc)
    state = ckpt.model_state_for_save(model)
    assert ("lm_head.weight" in state) != ("transformer.wte.weight" in state)      # stored once
    other = GPT(gc, tc)
    ckpt.load_model_state(other, dict(state))
    assert torch.equal(other.lm_head.weight, model.lm_head.weight)
    assert other.transformer.wte.weight.data_ptr() == other.lm_head.weight.data_ptr()


def test_pipeline_export_merges_and_renumbers(tmp_path):
    from gpt_moe_b200.checkpointing import checkpoint as ckpt
    from safetensors.torch import load_file
    gc, tc = tiny()
    torch.manual_seed(4)
    full = GPT(gc, tc)
    torch.manual_seed(4)
    s0, s1 = GPT(gc, tc, stage_index=0), None
    torch.manual_seed(4)
    s1 = GPT(gc, tc, stage_index=1)
    p0 = ckpt.save_stage_weights_for_export(s0, str(tmp_path), 3, 0)
    p1 = ckpt.save_stage_weights_for_export(s1, str(tmp_path), 3, 1)
    out = ckpt.export_full_model_pp([p0, p1], build_resume_config(gc, tc), str(tmp_path), 3, 256)
    merged = load_file(out)
    assert set(merged) == set(full.state_dict())
    assert torch.equal(merged["transformer.h.1.attn.q_proj.weight"], full.state_dict()["transformer.h.1.attn.q_proj.weight"])
    assert os.path.exists(os.path.join(str(tmp_path), "full_model_step_0000003_config.json"))
