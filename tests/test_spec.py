import os

import pytest

from parameter_golf_b200.spec import RunSpec, family_preset


def test_partial_toml_loads(tmp_path):
    f = tmp_path / "s.toml"
    f.write_text('name = "x"\nmode = "smoke"\n[model]\nnum_layers = 12\n[model.bigram]\nenabled = true\nvocab_size = 64\n[eval]\nstride = 32\n')
    s = RunSpec.load(str(f)).validate()
    assert s.model.num_layers == 12 and s.model.bigram.enabled and s.eval.stride == 32 and s.train.seq_len == 2048
    # what the file leaves out comes from the reference's default family (pg-model/src/spec.rs:693-697), nested tables included
    assert (s.model.family, s.model.vocab_size, s.model.bigram.vocab_size, s.model.bigram.dim) == ("baseline_sp8192", 8192, 64, 112)
    g = tmp_path / "t.toml"
    g.write_text('[model]\nfamily = "tiny_cpu"\nnum_layers = 3\n')
    t = RunSpec.load(str(g)).validate()
    assert t.model.num_layers == 3 and t.model.model_dim == family_preset("tiny_cpu").model.model_dim
    g.write_text('[model]\nfamily = "nope"\n')
    with pytest.raises(ValueError):
        RunSpec.load(str(g))


def test_the_reference_engines_shipped_spec_files_load(tmp_path):
    """The five spec files of the reference tree, restated here key for key where they matter (the files themselves are not
    part of this repository): every key they use is accepted, omitted keys fall back to baseline_sp8192."""
    frontier = tmp_path / "frontier.toml"
    frontier.write_text("""
name = "frontier_1855_merged_target"
mode = "smoke"
[model]
family = "frontier_1855_like"
attention_backend = "cudnn_sdpa_bf16"
compute_precision = "bf16_tensor_core"
mlp_mult = 4.0
xsa_last_n = 11
smear_gate_boundary_token_id = 1
[model.bigram]
enabled = false
vocab_size = 3072
dim = 112
[model.value_embedding]
enabled = false
dim = 128
layers = []
[model.recurrence]
enabled = true
start_layer = 4
repeat_layers = 2
[model.parallel_residual]
enabled = true
split_attention_mlp = true
[model.attn_out_gate]
enabled = false
width = 24
[model.caseops]
enabled = true
byte_sidecar = true
[model.sparse_attn_gate]
enabled = true
width = 12
scale = 0.5
[train]
backend = "cuda_distributed"
distributed_optimizer_backend = "sharded_parallel_muon"
batch_tokens = 786432
world_size = 8
fast_bank_updates = false
warmdown_frac = 0.85
min_lr_scale = 0.10
adam_beta2 = 0.99
[quant]
scheme = "mixed_int5_int6"
calibration = "self_generated"
compression = "pergroup"
embed_bits = 7
mlp_clip_sigmas = 11.5
gptq_calibration_batches = 16
[quant.lqer]
enabled = true
rank = 4
top_k = 3
a_bits = 2
b_bits = 4
group_size = 64
asymmetric = true
[eval]
qttt = true
adaptation_backend = "gpu_lora_phased"
lora_rank = 80
phased_ttt_prefix_docs = 2500
phased_ttt_weight_decay = 0.5
ttt_beta2 = 0.99
caseops_byte_sidecar_pattern = "data/fineweb_val_bytes_*.bin"
""")
    s = RunSpec.load(str(frontier)).validate()
    m = s.model
    assert m.parallel and m.caseops.byte_sidecar and not m.bigram.enabled and m.mlp_dim == 2048 and m.xsa_layers() == list(range(11))
    assert s.eval.lora_alpha == 144.0 and s.eval.phased_ttt_phases == 3 and s.quant.attn_clip_sigmas == 13.0        # left out: reference defaults
    smoke = tmp_path / "lora.toml"
    smoke.write_text('name = "baseline_gpu_lora_eval_smoke"\nmode = "smoke"\n[eval]\nstride = 512\nqttt = true\nadaptation_backend = "gpu_lora_phased"\n'
                     'lora_rank = 16\nlora_alpha = 16.0\nphased_ttt_phases = 2\nchunk_tokens = 4096\nmax_tokens = 4096\n')
    b = RunSpec.load(str(smoke)).validate()
    assert b.model.family == "baseline_sp8192" and b.model.value_embedding.enabled and b.model.qk_gain_init == 5.0 and b.eval.legal_score_first
    # enabled without the split flag is the sequential block, as in the reference (pg-model/src/spec.rs:421-422)
    seq = family_preset("parallel_resid_sp8192")
    seq.model.parallel_residual.split_attention_mlp = False
    assert not seq.model.parallel and family_preset("parallel_resid_sp8192").model.parallel
    with pytest.raises(ValueError):
        RunSpec.load(str(frontier)).apply_overrides(["mode=record", "eval.caseops_byte_sidecar_pattern=", "train.train_data_pattern=a", "train.validation_data_pattern=b"]).validate()


def test_unknown_key_rejected(tmp_path):
    f = tmp_path / "s.toml"
    f.write_text("[model]\nnot_a_key = 1\n")
    with pytest.raises(KeyError):
        RunSpec.load(str(f))


def test_toml_roundtrip():
    s = family_preset("record_11l")
    import tomllib
    s2 = RunSpec.from_dict(tomllib.loads(s.to_toml()))
    assert s2.to_dict() == s.to_dict()


def test_env_overlay_uses_train_gpt_names():
    s = family_preset("baseline_9l").apply_env({"NUM_LAYERS": "5", "TRAIN_SEQ_LEN": "512", "BIGRAM_VOCAB_SIZE": "3072",
                                                "XSA_LAST_N": "2", "MATRIX_LR": "0.01", "VE_LAYERS": "3,4", "TTT_ENABLED": "1"})
    assert s.model.num_layers == 5 and s.train.seq_len == 512 and s.model.train_seq_len == 512
    assert s.model.bigram.enabled and s.model.bigram.vocab_size == 3072 and s.model.xsa_last_n == 2
    assert s.train.matrix_lr == 0.01 and s.model.value_embedding.layers == [3, 4] and s.eval.legal_score_first


def test_overrides():
    s = family_preset("tiny_cpu").apply_overrides(["train.matrix_lr=0.5", "model.bigram.enabled=true", "eval.max_tokens=100"])
    assert s.train.matrix_lr == 0.5 and s.model.bigram.enabled is True and s.eval.max_tokens == 100
    with pytest.raises(KeyError):
        s.apply_overrides(["train.nope=1"])


@pytest.mark.parametrize("ov", ["model.num_heads=7", "model.rope.mode=spiral", "model.rope.yarn_max_len=0 model.rope.mode=yarn", "quant.compression=brotli", "train.rank=3",
                                "model.vocab_size=70000", "quant.matrix_bits=3", "train.batch_tokens=1000"])
def test_validation_rejects(ov):
    with pytest.raises(ValueError):
        family_preset("tiny_cpu").apply_overrides(ov.split()).validate()


def test_single_gpu_backends_reject_more_than_one_rank_but_cpu_runs_data_parallel():
    with pytest.raises(ValueError):
        family_preset("tiny_cpu").apply_overrides(["train.backend=cuda_single", "train.world_size=2"]).validate()
    family_preset("tiny_cpu").apply_overrides(["train.world_size=2", "train.rank=1"]).validate()      # gloo ranks on the CPU backend


def test_gates_mutually_exclusive():
    s = family_preset("tiny_cpu").apply_overrides(["model.attn_out_gate.enabled=true", "model.sparse_attn_gate.enabled=true"])
    with pytest.raises(ValueError):
        s.validate()


def test_record_mode_is_fail_closed():
    s = family_preset("record_11l")
    s.mode = "record"
    s.train.world_size = 8
    with pytest.raises(ValueError):
        s.validate()     # no data patterns
    s.allow_unsupported_variants = True
    s.validate()


def test_fingerprint_sensitivity():
    a = family_preset("record_11l").fingerprint()
    assert a == family_preset("record_11l").fingerprint()
    assert a != family_preset("record_11l").apply_overrides(["model.xsa_last_n=3"]).fingerprint()
    assert a != family_preset("record_11l").apply_overrides(["train.matrix_lr=0.03"]).fingerprint()
    assert a == family_preset("record_11l").apply_overrides(["train.train_log_every=7"]).fingerprint()


def test_presets_match_benchmark_configs():
    t = family_preset("tiny_cpu").validate().model
    assert (t.num_layers, t.model_dim, t.num_heads, t.num_kv_heads, t.head_dim, t.mlp_dim) == (2, 128, 4, 2, 32, 256)
    b = family_preset("baseline_9l").validate()
    assert (b.model.num_layers, b.model.rope_dims, b.train.batch_tokens, b.train.seq_len) == (9, 64, 524288, 1024)
    r = family_preset("record_11l").validate()
    assert (r.model.mlp_dim, r.model.rope_dims, r.model.xsa_layers(), r.model.bigram.vocab_size) == (1536, 16, [7, 8, 9, 10], 3072)
    assert r.train.distributed_optimizer_backend == "sharded_parallel_muon" and r.train.batch_tokens == 786432


def test_optional_record_ideas_are_cpu_only_and_read_from_the_environment():
    from parameter_golf_b200.spec import RunSpec
    s = family_preset("tiny_cpu").apply_overrides(["model.value_residual=true", "model.mtp_num_heads=2"]).validate()
    assert s.model.value_residual and s.model.mtp_num_heads == 2
    with pytest.raises(ValueError):
        family_preset("record_11l").apply_overrides(["model.value_residual=true"]).validate()
    with pytest.raises(ValueError):
        family_preset("record_11l").apply_overrides(["model.mtp_num_heads=1"]).validate()
    e = family_preset("tiny_cpu")
    e.apply_env({"VALUE_RESIDUAL": "1", "MTP_NUM_HEADS": "3", "MTP_LOSS_WEIGHT": "0.1", "ROPE_TYPE": "yarn", "YARN_MAX_LEN": "4096"})
    assert e.model.value_residual and e.model.mtp_num_heads == 3 and e.model.mtp_loss_weight == 0.1
    assert e.model.rope.mode == "yarn" and e.model.rope.yarn_max_len == 4096
    e.validate()


def test_binary_submission_environment_names():
    """run_cuda_binary.sh's names: ACTIVATION=relu2 / swiglu, SMEAR (the per-block running-mean smear), BITNET_GROUP_SIZE (both the
    trained and the stored group), WARMDOWN_FRACTION; the SwiGLU non-record run's MLP_HIDDEN, WARMDOWN_FRAC, GRAD_ACCUM_STEPS."""
    e = family_preset("tiny_cpu")
    e.apply_env({"ACTIVATION": "relu2", "SMEAR": "1", "BITNET_GROUP_SIZE": "64", "WARMDOWN_FRACTION": "0.2", "MODEL_DIM": "96", "MLP_HIDDEN": "200",
                 "GRAD_ACCUM_STEPS": "2"})
    assert e.model.activation == "relu_sq" and e.model.block_smear and e.model.qat_ternary_group == e.quant.ternary_group == 64
    assert e.train.warmdown_frac == 0.2 and e.model.mlp_dim == 200 and e.train.grad_accum_steps == 2
    e.apply_env({"ACTIVATION": "swiglu", "WARMDOWN_FRAC": "0.3"})
    assert e.model.activation == "swiglu" and e.train.warmdown_frac == 0.3
    e.validate()


def test_key_listing_and_environment_names_follow_the_code():
    """`describe_keys` walks the dataclasses; `env_names` is read off `apply_env` itself: every environment name maps to keys
    that exist, and setting the variable really changes one of them."""
    from parameter_golf_b200.spec import RunSpec
    keys = {k for k, _, _ in RunSpec().describe_keys()}
    assert {"model.num_layers", "model.rope.yarn_max_len", "train.lawa_k", "quant.float_storage", "eval.stride", "mode"} <= keys
    env = RunSpec.env_names()
    assert env["NUM_LAYERS"] == ["model.num_layers"] and env["TRAIN_SEQ_LEN"] == ["train.seq_len", "model.train_seq_len"]
    assert env["RUN_ID"] == ["name"] and "model.fp8_qat" in env["FP_STORAGE"]
    for name, mapped in env.items():
        assert mapped, name
        for k in mapped:
            assert k in keys, (name, k)
    sample = {"NUM_LAYERS": "7", "MUON_WD": "0.01", "EVAL_STRIDE": "32", "LAWA_K": "4"}
    before = dict((k, v) for k, _, v in RunSpec().describe_keys())
    after = dict((k, v) for k, _, v in RunSpec().apply_env(sample).describe_keys())
    for name in sample:
        assert any(before[k] != after[k] for k in env[name]), name


def test_keys_subcommand_prints_every_key(capsys):
    from parameter_golf_b200.train import main
    assert main(["keys"]) == 0
    out = capsys.readouterr().out
    assert "model.num_layers (int) = 11  env NUM_LAYERS" in out and "train.seq_len (int) = 2048  env TRAIN_SEQ_LEN  flag --seq-len" in out


def test_sweep_architectures_match_the_reference_table():
    """pg-model/src/arch.rs:137-168 and its tests (:46-85): baseline = 512 x 11 x 3 with XSA on the last four; wide has head_dim 72
    and kv_dim 288; full XSA covers all 11; deep-narrow is 16 x 384 with head_dim 64 and four XSA layers."""
    from parameter_golf_b200.spec import ARCH_VARIANTS, arch_label, arch_variant
    assert len(ARCH_VARIANTS) == 10
    b = arch_variant("baseline").validate().model
    assert (b.model_dim, b.num_layers, b.mlp_dim, b.rope_dims, b.xsa_last_n, b.train_seq_len, b.vocab_size) == (512, 11, 1536, 16, 4, 2048, 1024)
    w = arch_variant("wide").validate()
    assert w.model.head_dim == 72 and w.model.kv_dim == 288 and w.train.backend == "cpu"
    assert arch_variant("full_xsa").model.xsa_last_n == 11
    dn = arch_variant("deep_narrow").validate().model
    assert (dn.num_layers, dn.model_dim, dn.head_dim, dn.xsa_last_n, dn.rope_dims) == (16, 384, 64, 4, 12)
    assert arch_variant("long_ctx").train.seq_len == 4096 and arch_variant("high_gqa").model.head_dim == 40
    assert arch_label("baseline") == "d512_h8_kv4_L11_m3_r16_x7_s2048"
    with pytest.raises(ValueError):
        arch_variant("nope")
    for k in ARCH_VARIANTS:
        arch_variant(k).validate()


def test_spec_subcommand_writes_a_loadable_file_for_every_family(tmp_path, capsys):
    from parameter_golf_b200.spec import FAMILIES
    from parameter_golf_b200.train import main
    for fam in FAMILIES:
        assert main(["spec", "--family", fam]) == 0
        f = tmp_path / f"{fam}.toml"
        f.write_text(capsys.readouterr().out)
        assert RunSpec.load(str(f)).validate().fingerprint() == family_preset(fam).fingerprint(), fam
    assert main(["spec", "--family", "tiny_cpu", "model.num_layers=3"]) == 0
    assert "num_layers = 3" in capsys.readouterr().out
