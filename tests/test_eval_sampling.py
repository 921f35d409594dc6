"""Sampling, HellaSwag scoring, GSM8K extraction/generation and the BPE tokenizer on CPU with a tiny model."""
import json
import os
from decimal import Decimal
from types import SimpleNamespace

import contextlib
import pytest
import torch

from gpt_moe_b200.config import get_preset
from gpt_moe_b200.models.gpt import GPT
from gpt_moe_b200.tokenizer import ByteTokenizer, load_tokenizer
from gpt_moe_b200.tokenizer.bpe import BytePairEncoding


def _run(tmp_path=None):
    gc, tc = get_preset("tiny_cpu")
    gc.n_layers, gc.vocab_size, gc.weighted_main_path_init = 1, 512, 0.5
    gc.pad_token_id, gc.eos_token_id = 511, 510
    tc.seq_len_train = tc.seq_len_val = 512
    tc.resolve(1)
    torch.manual_seed(0)
    model = GPT(gc, tc).eval()
    model.set_sliding_window(512)
    run = SimpleNamespace(parallel_mode="ddp", rank=0, world_size=1, master_process=True, device="cpu", training_config=tc,
                          gpt_model=model, raw_gpt_model=model, tokenizer=ByteTokenizer(), ctx=contextlib.nullcontext(), log_buffer=[],
                          forward=lambda m, ids, targets=None, attn_mask=None, ignore_doc_mask=False, document_ids=None:
                          m(ids, targets, attn_mask=attn_mask, ignore_doc_mask=ignore_doc_mask, document_ids=document_ids))
    return run


def test_bpe_roundtrip_and_merges():
    bpe = BytePairEncoding()
    text = "the quick brown fox jumps over the lazy dog; the the the quick quick"
    bpe.train(text, 300)
    assert bpe.n_vocab > 256
    ids = bpe.encode(text)
    assert len(ids) < len(text.encode()) and bpe.decode(ids) == text
    assert bpe.decode(bpe.encode("unseen żółć")) == "unseen żółć"
    assert isinstance(load_tokenizer("bytes"), ByteTokenizer)


def test_sampling_filters_and_generation_length():
    from gpt_moe_b200.sampling.sample import filter_logits, get_sample_token_count, sample
    logits = torch.tensor([[1.0, 3.0, 2.0, 0.0]])
    assert torch.isinf(filter_logits(logits, 2, None)).sum() == 2
    kept = ~torch.isinf(filter_logits(logits, None, 0.6))
    assert kept[0, 1] and kept.sum() <= 2
    assert get_sample_token_count(0) == 5 and get_sample_token_count(2500) == 15 and get_sample_token_count(10 ** 6) == 50
    run = _run()
    torch.manual_seed(1)
    out = sample(run, ["ab", "hello"], max_new_tokens=4, temperature=0.8, top_k=20)
    assert len(out) == 2 and out[1].startswith("hello")
    greedy_a = sample(run, ["xyz"], max_new_tokens=3, temperature=0.0)
    greedy_b = sample(run, ["xyz"], max_new_tokens=3, temperature=0.0)
    assert greedy_a == greedy_b


def test_hellaswag_scoring_and_evaluation(tmp_path, monkeypatch):
    from gpt_moe_b200.evaluation import hellaswag as hs
    # length-normalised continuation score: position j predicts token j+1
    logits = torch.full((1, 4, 5), -10.0)
    ids = torch.tensor([[1, 2, 3, 4]])
    logits[0, 1, 3] = 10.0
    logits[0, 2, 4] = 10.0
    score = hs.continuation_scores(logits, ids, [2], [4])
    assert score.item() == pytest.approx(0.0, abs=1e-3)
    rows = [{"ctx": f"context {i}", "endings": [f"end a{i}", f"end b{i}", f"end c{i}", f"end d{i}"], "label": i % 4} for i in range(6)]
    for name in ("hellaswag_train.jsonl", "hellaswag_val.jsonl"):
        with open(tmp_path / name, "w") as f:
            f.write("\n".join(json.dumps(r) for r in rows))
    monkeypatch.setenv("HELLASWAG_DIR", str(tmp_path))
    run = _run()
    hs.load_hellaswag_data(run)
    assert len(run.local_hellaswag_val_dataset) == 6
    acc = hs.evaluate_hellaswag_standard(run, hellaswag_examples_per_batch=4)
    assert 0.0 <= acc <= 1.0
    acc2 = hs.evaluate_hellaswag_one_shot(run, hellaswag_examples_per_batch=3)
    assert 0.0 <= acc2 <= 1.0


def test_gsm8k_extraction_and_generation(tmp_path, monkeypatch):
    from gpt_moe_b200.evaluation import gsm8k
    assert gsm8k.extract_gsm8k_answer("so\n#### 1,234.50\n") == Decimal("1234.50")
    assert gsm8k.extract_gsm8k_answer("#### -7") == Decimal("-7")
    assert gsm8k.extract_gsm8k_answer("the answer is 7") is None
    rows = [{"question": f"What is {i}+{i}?", "answer": f"<<{i}+{i}={2*i}>>It is {2*i}.\n#### {2*i}"} for i in range(1, 5)]
    for name in ("train.jsonl", "test.jsonl"):
        with open(tmp_path / name, "w") as f:
            f.write("\n".join(json.dumps(r) for r in rows))
    monkeypatch.setenv("GSM8K_DIR", str(tmp_path))
    run = _run()
    run.training_config.gsm8k_num_shots, run.training_config.gsm8k_max_new_tokens = 1, 6
    run.training_config.gsm8k_max_examples, run.training_config.gsm8k_examples_per_batch = 3, 2
    gsm8k.load_gsm8k_data(run)
    assert len(run.local_gsm8k_examples) == 3 and run.local_gsm8k_examples[0][1] == Decimal(2)
    assert "<<" not in run.tokenizer.decode(run.local_gsm8k_examples[0][0])
    acc = gsm8k.evaluate_gsm8k(run)
    assert 0.0 <= acc <= 1.0
    run.training_config.gsm8k_max_new_tokens = 10 ** 6
    with pytest.raises(ValueError, match="exceed max_seq_len"):
        gsm8k.load_gsm8k_data(run)


def test_validation_and_full_fit_loop_on_cpu(tmp_path):
    """`Trainer.fit` end to end on CPU: warm-up + restore, logging, validation, checkpoint, export, resume."""
    from dist_helpers import free_port
    from gpt_moe_b200.runtime.trainer import Trainer
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(free_port()), RANK="0", WORLD_SIZE="1", LOCAL_RANK="0")
    gc, tc = get_preset("tiny_cpu")
    gc.n_layers, gc.vocab_size = 1, 512
    tc.seq_len_train = tc.seq_len_val = 64
    tc.val_tokens = 2 * 4 * 64
    tc.enable_checkpointing, tc.checkpoint_interval, tc.export_full_model_at_end = True, 2, True
    tc.checkpoint_dir, tc.model_export_dir = str(tmp_path / "ckpt"), str(tmp_path / "export")
    tc.config_and_log_dir = str(tmp_path / "logs")
    tc.log_filename, tc.config_filename = str(tmp_path / "logs" / "log.txt"), str(tmp_path / "logs" / "config.txt")
    tc.max_tokens = 4 * 4 * 64
    trainer = Trainer(gc, tc, device_type="cpu", quiet=True)
    before = {n: p.detach().clone() for n, p in trainer.raw_gpt_model.named_parameters()}
    trainer.fit()
    assert any((p.detach() != before[n]).any() for n, p in trainer.raw_gpt_model.named_parameters())
    files = sorted(os.listdir(tmp_path / "ckpt"))
    assert any(f.startswith("model_step_0000003") for f in files) and "training_state_step_0000003.pt" in files
    assert os.path.exists(tmp_path / "export" / "full_model_step_0000003.safetensors")
    log = open(tmp_path / "logs" / "log.txt").read()
    assert "train loss" in log and "val loss" in log and "kernel warmup" in log
    weights = [f for f in files if f.startswith("model_step_0000003")][0]
    final = {n: p.detach().clone() for n, p in trainer.raw_gpt_model.named_parameters()}
    trainer.close()

    gc2, tc2 = get_preset("tiny_cpu")
    gc2.n_layers, gc2.vocab_size = 1, 512
    tc2.seq_len_train = tc2.seq_len_val = 64
    tc2.val_tokens, tc2.max_tokens = 2 * 4 * 64, 6 * 4 * 64
    tc2.resume_from_checkpoint = True
    tc2.resume_checkpoint_path = str(tmp_path / "ckpt" / weights)
    tc2.resume_state_dict_path = str(tmp_path / "ckpt" / "training_state_step_0000003.pt")
    tc2.export_full_model_at_end = False
    tc2.config_and_log_dir = str(tmp_path / "logs2")
    tc2.log_filename, tc2.config_filename = str(tmp_path / "logs2" / "log.txt"), str(tmp_path / "logs2" / "config.txt")
    os.environ["MASTER_PORT"] = str(free_port())
    with pytest.raises(ValueError, match="configuration differs"):     # max_tokens feeds the schedules: a different run
        Trainer(gc2, tc2, device_type="cpu", quiet=True)
    tc2.max_tokens = 4 * 4 * 64
    tc2.resolve(1)
    resumed = Trainer(gc2, tc2, device_type="cpu", quiet=True)
    assert resumed.start_step == 4 and resumed.train_tokens_processed == 4 * 4 * 64
    for n, p in resumed.raw_gpt_model.named_parameters():
        assert torch.equal(p.detach(), final[n]), n
    resumed.close()
