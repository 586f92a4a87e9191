"""fc_llama_load_gguf / fc_llama_gguf_probe against files written by ferrum_cpu_b200.gguf_file:
the keys, defaults and refusals of Gguf::load_llama (gguf/llama.rs:164-339). Probing needs no GPU;
loading is compared with the model built from the same arrays."""
import numpy as np
import pytest

from ferrum_cpu_b200 import _lib, gguf_file, llama, synth
from ferrum_cpu_b200.engine import FerrumCudaError

VT_U32, VT_F32, VT_STRING = gguf_file.VT_U32, gguf_file.VT_F32, gguf_file.VT_STRING


def tiny(**kw):
    return synth.llama_named("llama-tiny", perturb=True, **kw)


def test_probe_reads_the_configuration(tmp_path):
    sm = tiny(freq_factors=[1.0, 4.0] * 4, rope_linear_factor=2.0, rope_dim=16, norm_eps=1e-5)
    cfg = llama.gguf_probe(gguf_file.write_llama_gguf(tmp_path / "m.gguf", sm))
    want = sm.config
    for k in ("vocab", "d_model", "n_layer", "n_head", "n_kv_head", "head_dim", "d_ff", "rope_dim", "ctx", "tied"):
        assert getattr(cfg, k) == getattr(want, k), k
    assert cfg.rope_type == _lib.FC_ROPE_NORM and cfg.rope_linear_factor == 2.0
    assert abs(cfg.norm_eps - 1e-5) < 1e-12 and cfg.rope_base == 10000.0
    # qwen2 files rotate split halves, carry q/k/v biases and often an untied head (gguf/llama.rs:181-186)
    sq = tiny(rope_type=1, qkv_bias=True, tied=False, rope_base=1000000.0)
    cq = llama.gguf_probe(gguf_file.write_llama_gguf(tmp_path / "q.gguf", sq, arch="qwen2"))
    assert cq.rope_type == _lib.FC_ROPE_NEOX and cq.tied == 0 and cq.rope_base == 1000000.0


def test_defaults_when_keys_are_absent(tmp_path):
    sm = tiny()
    drop = ("llama.attention.head_count_kv", "llama.attention.key_length", "llama.rope.dimension_count", "llama.rope.freq_base",
            "llama.attention.layer_norm_rms_epsilon", "llama.context_length")
    # without head_count_kv the heads are not grouped, so the k / v projections of this file no longer fit
    with pytest.raises(FerrumCudaError) as e:
        llama.gguf_probe(gguf_file.write_llama_gguf(tmp_path / "a.gguf", sm, drop_meta=drop))
    assert e.value.code == _lib.FC_E_FORMAT and "attn_k.weight" in str(e.value)
    cfg = llama.gguf_probe(gguf_file.write_llama_gguf(tmp_path / "b.gguf", sm, drop_meta=drop[1:]))
    assert cfg.head_dim == 16 and cfg.rope_dim == 16 and cfg.rope_base == 10000.0 and cfg.ctx == 2048
    assert abs(cfg.norm_eps - 1e-5) < 1e-12


def test_refusals(tmp_path):
    sm = tiny()

    def refuse(name, text, **kw):
        with pytest.raises(FerrumCudaError) as e:
            llama.gguf_probe(gguf_file.write_llama_gguf(tmp_path / name, sm, **kw))
        assert e.value.code == _lib.FC_E_FORMAT and text in str(e.value), str(e.value)

    refuse("arch.gguf", "llama / qwen2 only", arch="gpt2")
    refuse("yarn.gguf", "yarn", extra_meta=[("llama.rope.scaling.type", VT_STRING, "yarn")])
    refuse("none.gguf", "\"none\" but the scaling factor", extra_meta=[("llama.rope.scaling.type", VT_STRING, "none"),
                                                                   ("llama.rope.scaling.factor", VT_F32, 4.0)])
    refuse("attn.gguf", "attn_factor", extra_meta=[("llama.rope.scaling.attn_factor", VT_F32, 0.5)])
    refuse("bias.gguf", "ffn_up.bias", extra_tensors=[("blk.0.ffn_up.bias", np.zeros(128, np.float32), (128,))])
    refuse("obias.gguf", "output.bias", extra_tensors=[("output.bias", np.zeros(512, np.float32), (512,))])
    # the legacy linear key, a factor of 0 (none) and "none" with factor 1 are accepted (gguf/llama.rs:520-545)
    for i, (meta, want) in enumerate([([("llama.rope.scale_linear", VT_F32, 2.0)], 2.0), ([("llama.rope.scaling.factor", VT_F32, 0.0)], 1.0),
                                      ([("llama.rope.scaling.type", VT_STRING, "none")], 1.0), ([("llama.rope.scaling.factor", VT_F32, 4.0)], 4.0)]):
        cfg = llama.gguf_probe(gguf_file.write_llama_gguf(tmp_path / f"ok{i}.gguf", sm, extra_meta=meta))
        assert cfg.rope_linear_factor == want


@pytest.mark.gpu
@pytest.mark.parametrize("arch,kw", [("llama", dict(freq_factors=[1.0, 4.0] * 4, rope_linear_factor=2.0)),
                                      ("qwen2", dict(rope_type=1, qkv_bias=True, tied=False))])
def test_model_from_file_equals_model_from_arrays(tmp_path, arch, kw):
    sm = tiny(**kw)
    path = gguf_file.write_llama_gguf(tmp_path / "m.gguf", sm, arch=arch)
    a, b = llama.CudaLlama.from_synth(sm), llama.CudaLlama.from_gguf(path)
    ids = synth.token_ids(5, 40, sm.dims["vocab"])
    assert np.array_equal(a.forward_tokens(ids), b.forward_tokens(ids))
    ca, cb = a.new_cache(), b.new_cache()
    for t in ids[:6]:
        assert np.array_equal(a.forward_one(t, ca), b.forward_one(t, cb))
    capped = llama.CudaLlama.from_gguf(path, ctx_cap=16)
    assert capped.config.ctx == 16
    with pytest.raises(FerrumCudaError):
        capped.score_from(ids, 1, 32)
    for m in (a, b, capped):
        m.close()
