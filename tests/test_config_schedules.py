import math

import pytest

from gpt_moe_b200.config import TrainingConfig, apply_overrides, build_resume_config, get_preset
from gpt_moe_b200.schedules import token as sched


def test_lr_schedule_shape():
    kw = dict(lr_warmup_tokens=100, lr_warmup_and_cosine_tokens=1100, total_decay_tokens=1000, adamw_max_lr=1.0, adamw_hard_min_lr=0.1)
    assert sched.get_token_based_adamw_lr(0, **kw) == pytest.approx(1 / 100)
    assert sched.get_token_based_adamw_lr(100, **kw) == pytest.approx(1.0)
    assert sched.get_token_based_adamw_lr(600, **kw) == pytest.approx(0.1 + 0.5 * 0.9)
    assert sched.get_token_based_adamw_lr(1100, **kw) == 0.1
    assert sched.get_token_based_adamw_lr(10 ** 9, **kw) == 0.1


def test_schedule_generators():
    assert sched.add_schedule(128, 128, count=3) == [128, 256, 384]
    assert sched.add_schedule(1, 2, end=6) == [1, 3, 5]
    assert sched.factor_schedule(2, 2, count=4) == [2, 4, 8, 16]
    assert sched.factor_schedule(3, 2, end=20) == [3, 6, 12]
    assert sched.custom_schedule([4, 8]) == [4, 8]
    assert sched.enforce_min_max_constraints([5, 3, 9, 20], 4, 10) == [5, 5, 9, 10]
    assert sched.enforce_flex_block_constraints(300, 128, False) == 256
    assert sched.enforce_flex_block_constraints(100, 128, False) == 128
    assert sched.enforce_flex_block_constraints(384, 128, True) == 512
    assert sched.get_next_update_tokens([0, 50], 0, 99) == 50
    assert sched.get_next_update_tokens([10, 50], 0, 99) == 10
    assert sched.get_next_update_tokens([0, 50], 1, 99) == 100


def test_default_resolve_matches_reference_derivations():
    tc = TrainingConfig()
    tc.resolve(4)
    assert tc.total_tokens_per_mini_step_train == 4 * 8 * 8192
    assert tc.grad_accum_mini_steps == 1
    assert tc.val_steps == math.ceil(5 * 2 ** 21 / (4 * 8 * 8192))
    assert tc.swa_schedule_values == [128 * i for i in range(1, 12)]
    assert tc.swa_schedule_keys[0] == 32_768_000 and len(tc.swa_schedule_keys) == 11
    assert tc.batch_size_schedule_keys == [0, 78_643_200] and tc.batch_size_schedule_values == [4, 8]
    assert tc.torch_compile_mode == "max-autotune"
    assert tc.max_train_steps == 5 * 10 ** 9 // 2 ** 18
    tc2 = TrainingConfig()
    tc2.resolve(1)
    assert tc2.grad_accum_mini_steps == 4 and tc2.torch_compile_mode == "max-autotune-no-cudagraphs"
    with pytest.raises(AssertionError):
        TrainingConfig(muon_backend_steps=4).resolve(1)


def test_presets_and_overrides():
    gc, tc = get_preset("small")
    assert (gc.n_layers, gc.hidden_size, gc.num_experts, gc.mlp_hidden_dim, gc.activation) == (12, 768, 8, 3072, "swiglu")
    tc.resolve(8)
    assert tc.grad_accum_mini_steps == 1 and tc.swa_schedule_values == [1024]
    gc, tc = get_preset("wide_ep")
    assert gc.num_experts == 32 and gc.moe_top_k == 2 and tc.expert_parallel_size == 8
    gc, tc = get_preset("mla")
    assert gc.use_mla and gc.moe_shared_expert_hidden_dim == 2048 and gc.num_experts == 64
    apply_overrides(gc, tc, ["model.n_layers=3", "training.seq_len_train=128", "training.muon_backend=svd"])
    assert gc.n_layers == 3 and tc.seq_len_train == 128 and tc.muon_backend == "svd"
    with pytest.raises(ValueError):
        apply_overrides(gc, tc, ["model.nope=1"])


def test_resume_config_keys():
    gc, tc = get_preset("tiny_cpu")
    tc.resolve(1)
    rc = build_resume_config(gc, tc)
    assert set(rc) >= {"model", "training", "bf16_weights_params_and_scales", "lr_schedule"}
    assert rc["lr_schedule"][0]["fn"] == "get_token_based_adamw_lr"
    assert rc["training"]["linear_config"]["training"]["q_proj"]["precision"] == "default"


def test_linear_config_validation():
    from gpt_moe_b200.models.gpt import GPT
    gc, tc = get_preset("tiny_cpu")
    tc.resolve(1)
    tc.linear_config["training"]["router"]["precision"] = "fp8"
    with pytest.raises(ValueError, match="router"):
        GPT(gc, tc)
    tc.linear_config["training"]["router"]["precision"] = "bogus"
    with pytest.raises(ValueError, match="unsupported linear precision"):
        GPT(gc, tc)
