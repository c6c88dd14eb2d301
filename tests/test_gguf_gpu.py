"""GGUF file -> device model: files written with the `gguf` Python package (the published format's own
writer) are read by the library's loader; configuration, tensor bytes and greedy tokens must match the
model the file was written from."""
import os

import numpy as np
import pytest

import densecore_b200 as dc
from densecore_b200 import blocks as B

gguf = pytest.importorskip("gguf")
pytestmark = pytest.mark.gpu


def write_gguf(path, m: dc.Model, arch: str, drop=(), extra_meta=True, moe_meta=None):
    cfg = m.cfg
    w = gguf.GGUFWriter(path, arch)
    w.add_block_count(cfg.n_layer)
    w.add_embedding_length(cfg.hidden)
    w.add_head_count(cfg.n_head)
    w.add_head_count_kv(cfg.n_kv_head)
    w.add_key_length(cfg.head_dim)
    w.add_layer_norm_rms_eps(cfg.rms_eps)
    w.add_rope_freq_base(cfg.rope_theta)
    w.add_context_length(cfg.max_ctx)
    if cfg.n_expert:
        w.add_expert_count(cfg.n_expert)
        w.add_expert_used_count(cfg.n_expert_used)
        w.add_expert_feed_forward_length(cfg.expert_ffn)
    else:
        w.add_feed_forward_length(cfg.ffn)
    for key, val in (moe_meta or {}).items():   # <arch>.<key>, the MoE switches the reference's loader reads
        if isinstance(val, bool):
            w.add_bool(f"{arch}.{key}", val)
        elif isinstance(val, float):
            w.add_float32(f"{arch}.{key}", val)
        else:
            w.add_uint32(f"{arch}.{key}", val)
    if extra_meta:   # values the loader must step over
        w.add_array("tokenizer.ggml.tokens", [f"tok{i}" for i in range(50)])
        w.add_array("tokenizer.ggml.scores", [float(i) for i in range(50)])
        w.add_bool("general.some_flag", True)
    tensors = {}
    for name in m.tensor_names():
        if name in drop:
            continue
        t, (K, N, E), data = m.get_tensor(name)
        tensors[name] = (t, data.copy())
        if t == B.GGML_TYPE_F32:
            arr = data.reshape((N, K) if N > 1 else (K,))
            w.add_tensor(name, arr)
        else:
            rb = B.row_bytes(t, K)
            shape = (E, N, rb) if E > 1 else (N, rb)
            w.add_tensor(name, data.reshape(shape), raw_dtype=gguf.GGMLQuantizationType(t))
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    return tensors


@pytest.mark.parametrize("moe", [True, False])
def test_gguf_round_trip(ctx, tmp_path, moe):
    cfg = dc.Config(n_layer=2, hidden=512, n_head=4, n_kv_head=2, vocab=1000, max_seqs=2, max_ctx=64,
                    **(dict(n_expert=8, n_expert_used=2, expert_ffn=256) if moe else dict(ffn=768, tie_embeddings=True)))
    src = dc.Model(ctx, cfg)
    src.init_synthetic(11, 0.05)
    src.finalize()
    path = str(tmp_path / "model.gguf")
    tensors = write_gguf(path, src, "qwen3moe" if moe else "qwen3")
    m = dc.Model.from_gguf(ctx, path, max_seqs=2)
    for f in ("n_layer", "hidden", "n_head", "n_kv_head", "head_dim", "vocab", "ffn", "n_expert", "n_expert_used",
              "expert_ffn", "tie_embeddings", "qk_norm", "max_ctx"):
        assert getattr(m.cfg, f) == getattr(cfg, f), f
    assert abs(m.cfg.rms_eps - cfg.rms_eps) < 1e-12 and m.cfg.rope_theta == cfg.rope_theta
    m.finalize()
    for name, (t, data) in tensors.items():
        t2, _, d2 = m.get_tensor(name)
        assert t2 == t and np.array_equal(d2, data), name
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, cfg.vocab, size=21)
    outs = []
    for model in (src, m):
        s = model.seq_alloc()
        first, lg = model.prefill(s, prompt, want_logits=True)
        run, _ = model.decode_run([s], [first], 8)
        outs.append((first, lg, run))
    assert outs[0][0] == outs[1][0] and np.array_equal(outs[0][1], outs[1][1]) and np.array_equal(outs[0][2], outs[1][2])
    m.close()
    src.close()


def test_gguf_errors(ctx, tmp_path):
    cfg = dc.Config(n_layer=1, hidden=512, n_head=4, n_kv_head=2, vocab=300, ffn=512, tie_embeddings=True, max_seqs=1,
                    max_ctx=32)
    src = dc.Model(ctx, cfg)
    src.init_synthetic(3, 0.05)
    src.finalize()
    missing = str(tmp_path / "missing.gguf")
    write_gguf(missing, src, "qwen3", drop=("blk.0.attn_v.weight",), extra_meta=False)
    with pytest.raises(dc.DcError) as e:
        dc.Model.from_gguf(ctx, missing)
    assert e.value.status == -2 and "blk.0.attn_v.weight" in str(e.value)
    junk = tmp_path / "junk.gguf"
    junk.write_bytes(b"not a gguf file at all, just bytes" * 4)
    with pytest.raises(dc.DcError) as e:
        dc.Model.from_gguf(ctx, str(junk))
    assert e.value.status == -2
    good = str(tmp_path / "good.gguf")
    write_gguf(good, src, "qwen3")
    cut = tmp_path / "cut.gguf"
    cut.write_bytes(open(good, "rb").read()[:-4096])
    with pytest.raises(dc.DcError) as e:
        dc.Model.from_gguf(ctx, str(cut))
    assert e.value.status == -2
    with pytest.raises(dc.DcError):
        dc.Model.from_gguf(ctx, str(tmp_path / "absent.gguf"))
    src.close()


def test_gguf_moe_variants_the_decoder_does_not_compute_are_refused(ctx, tmp_path):
    """The reference's loader reads norm_topk_prob, shared experts, grouped routing and leading dense layers
    (core/src/models/model_loader.cpp:2833-2850); this decoder computes none of them, so such files fail with
    UNSUPPORTED instead of decoding wrong tokens.  routed_scaling_factor is accepted as the scale's other name."""
    cfg = dc.Config(n_layer=1, hidden=512, n_head=4, n_kv_head=2, vocab=300, n_expert=8, n_expert_used=2, expert_ffn=256,
                    max_seqs=1, max_ctx=32)
    src = dc.Model(ctx, cfg)
    src.init_synthetic(3, 0.05)
    src.finalize()
    for i, meta in enumerate(({"norm_topk_prob": False}, {"n_shared_experts": 1}, {"expert_shared_count": 2},
                              {"n_group": 4, "topk_group": 2}, {"first_k_dense_replace": 1}, {"leading_dense_block_count": 1})):
        path = str(tmp_path / f"variant{i}.gguf")
        write_gguf(path, src, "qwen3moe", extra_meta=False, moe_meta=meta)
        with pytest.raises(dc.DcError) as e:
            dc.Model.from_gguf(ctx, path)
        assert e.value.status == -7, (meta, e.value.status)
    ok = str(tmp_path / "scaled.gguf")
    write_gguf(ok, src, "qwen3moe", extra_meta=False, moe_meta={"routed_scaling_factor": 2.5, "norm_topk_prob": True})
    m = dc.Model.from_gguf(ctx, ok, max_seqs=1, max_ctx=32)
    assert abs(m.cfg.routed_scale - 2.5) < 1e-6
    m.close()
    src.close()
