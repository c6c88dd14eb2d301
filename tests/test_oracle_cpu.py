"""CPU tests: the oracle against golden vectors, known answers and independent
restatements.  No GPU needed."""
import os

import numpy as np
import pytest

from densecore_b200 import blocks as B

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "kquant_golden.npz"))


def test_philox_known_answers(oracle):
    # Philox4x32-10 known-answer vectors of the Random123 distribution (zero and pi-digit inputs)
    assert [hex(v) for v in oracle.philox4x32_10([0, 0, 0, 0], [0, 0])] == \
        ["0x6627e8d5", "0xe169c58d", "0xbc57ac4c", "0x9b00dbd8"]
    assert [hex(v) for v in oracle.philox4x32_10([0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344],
                                                 [0xa4093822, 0x299f31d0])] == \
        ["0xd16cfe09", "0x94fdcceb", "0x5001e420", "0x24126ea1"]
    assert np.array_equal(oracle.verify_uniforms(99, 3, 5), GOLD["uniforms_99_3"])


def test_fp16_conversions_match_numpy(oracle):
    h = np.arange(0, 65536, 13, dtype=np.uint16)
    f = h.view(np.float16).astype(np.float32)
    for hv, fv in zip(h.tolist(), f.tolist()):
        v = oracle.fp16_to_fp32(hv)
        assert (np.isnan(v) and np.isnan(fv)) or v == fv
    rng = np.random.default_rng(5)
    xs = (rng.normal(size=4000) * 10.0 ** rng.integers(-9, 5, size=4000)).astype(np.float32)
    with np.errstate(over="ignore"):
        want = xs.astype(np.float16).view(np.uint16)
    for x, w in zip(xs.tolist(), want.tolist()):
        assert oracle.fp32_to_fp16(x) == w


def test_q8k_quantiser_golden_and_semantics(oracle):
    q = oracle.quantize_q8k(GOLD["x"])
    assert np.array_equal(q, GOLD["q8_x"])
    assert np.array_equal(oracle.quantize_q8k(GOLD["x_pat"]), GOLD["q8_x_pat"])
    d, qs, bs = oracle.q8k_fields(q)
    # all-zero block -> zeros
    assert d[1, 1] == 0 and not qs[1, 1].any() and not bs[1, 1].any()
    # the largest-magnitude element maps to -127 and d has the opposite sign of it
    assert qs[2, 0, 7] == -127 and d[2, 0] > 0
    # bsums are sums of 16
    assert np.array_equal(bs, qs.reshape(3, 2, 16, 16).sum(-1).astype(np.int16))
    # independent numpy restatement of the rounding rule (round half to even, clip above only)
    x = GOLD["x"][0, :256]
    i = np.argmax(np.abs(x))
    iscale = np.float32(-127.0) / x[i]
    want = np.minimum(127, np.rint((iscale * x).astype(np.float32))).astype(np.int8)
    assert np.array_equal(qs[0, 0], want)


def test_q8k_first_of_equal_magnitudes_wins(oracle):
    x = np.zeros((1, 256), np.float32)
    x[0, 10], x[0, 200] = 3.0, -3.0
    _, qs, _ = oracle.q8k_fields(oracle.quantize_q8k(x))
    assert qs[0, 0, 10] == -127 and qs[0, 0, 200] == 127
    x[0, 10], x[0, 200] = -3.0, 3.0
    _, qs, _ = oracle.q8k_fields(oracle.quantize_q8k(x))
    assert qs[0, 0, 10] == -127 and qs[0, 0, 200] == 127


@pytest.mark.parametrize("name,t", [("q4k", B.GGML_TYPE_Q4_K), ("q6k", B.GGML_TYPE_Q6_K)])
def test_block_decode_and_dots_golden(oracle, name, t):
    w, N, K = GOLD[f"w_{name}"], 6, 512
    assert np.array_equal(oracle.dequantize(t, w, N, K), GOLD[f"deq_{name}"])  # == gguf.quants.dequantize
    y = oracle.mul_mat(t, w, N, K, GOLD["x"])
    assert np.array_equal(y, GOLD[f"y_{name}"])
    # integer block sums against a plain numpy restatement from the decoded integers
    rb = B.row_bytes(t, K)
    d8, q8, bs8 = oracle.q8k_fields(GOLD["q8_x"])
    for m in range(3):
        for n in range(N):
            I, M = oracle.block_sums(t, w.reshape(N, rb)[n], GOLD["q8_x"][m], K)
            assert np.array_equal(I, GOLD[f"I_{name}"][m, n])
            if M is not None:
                assert np.array_equal(M, GOLD[f"M_{name}"][m, n])
    # float result vs float64 dot of dequantised weights and dequantised activations
    act = (q8.astype(np.float64) * d8[..., None].astype(np.float64)).reshape(3, K)
    want = act @ GOLD[f"deq_{name}"].astype(np.float64).T
    assert np.abs(y - want).max() <= 1e-4 * np.abs(want).max()


def test_q4k_scale_packing_round_trip(oracle):
    rng = np.random.default_rng(3)
    sc = rng.integers(0, 64, size=(50, 8), dtype=np.uint8)
    mn = rng.integers(0, 64, size=(50, 8), dtype=np.uint8)
    packed = B.pack_q4k_scales(sc, mn)
    import ctypes as C
    for i in range(50):
        out = np.zeros(16, np.uint8)
        oracle.lib().dco_q4k_decode_scales(packed[i].ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p))
        assert np.array_equal(out[:8], sc[i]) and np.array_equal(out[8:], mn[i])


def test_router_golden_and_tie_rule(oracle):
    ids, w = oracle.route(GOLD["route_logits"], 4, mode="stable")
    assert np.array_equal(ids, GOLD["route_ids"]) and np.array_equal(w, GOLD["route_w"])
    # equal logits: the lower expert id comes first (core/src/llm/moe/native.cpp:610-620)
    row = GOLD["route_ids"][1].tolist()
    if 3 in row and 9 in row:
        assert row.index(3) < row.index(9)
    # generic softmax->top-k->renormalise route selects the same experts and weights (to rounding)
    ids2, w2 = oracle.route(GOLD["route_logits"], 4, mode="softmax")
    assert np.array_equal(ids2, ids)
    assert np.allclose(w2, w, rtol=1e-5)
    assert np.allclose(w.sum(1), 1.0, atol=1e-6)
    # numpy restatement
    lg = GOLD["route_logits"].astype(np.float64)
    for t in range(lg.shape[0]):
        order = sorted(range(16), key=lambda e: (-lg[t, e], e))[:4]
        assert order == ids[t].tolist()


def test_reorder_map_is_stable_grouping(oracle):
    ids = np.array([[3, 1], [1, 2], [3, 0]], np.int32)
    off, tok, slot = oracle.build_reorder_map(ids, 4)
    assert off.tolist() == [0, 1, 3, 4, 6]
    assert tok.tolist() == [2, 0, 1, 1, 0, 2]
    assert slot.tolist() == [5, 1, 2, 3, 0, 4]


def test_moe_quantised_path_close_to_f32_reference(oracle):
    """The reference's own probe tolerance between its quantised MoE path and its f32
    oracle is 1e-2 (core/src/backend/cpu_backend_moe_reference.inl:370-384)."""
    rng = np.random.default_rng(11)
    H, F, E, K, T = 512, 256, 8, 2, 3
    gate, up = B.random_q4k(rng, E * F, H, 0.002), B.random_q4k(rng, E * F, H, 0.002)
    down = B.random_q6k(rng, E * H, F, 0.002)
    x = rng.normal(size=(T, H)).astype(np.float32)
    ids, w = oracle.route(rng.normal(size=(T, E)).astype(np.float32), K)
    types = (B.GGML_TYPE_Q4_K, B.GGML_TYPE_Q4_K, B.GGML_TYPE_Q6_K)
    y = oracle.moe_forward(types, gate, up, down, E, H, F, x, ids, w, fast_exp=True)
    y_exp = oracle.moe_forward(types, gate, up, down, E, H, F, x, ids, w, fast_exp=False)
    y_ref = oracle.moe_forward(types, gate, up, down, E, H, F, x, ids, w, f32ref=True)
    scale = np.abs(y_ref).max()
    assert np.abs(y - y_exp).max() <= 2e-3 * scale      # polynomial exp vs std::exp
    assert np.abs(y - y_ref).max() <= 3e-2 * scale      # Q8_K activations vs f32 activations


def test_fast_exp_forms(oracle):
    xs = np.linspace(-30, 10, 401, dtype=np.float32)
    for x in xs.tolist():
        e = np.exp(np.float64(np.float32(x)))
        assert abs(oracle.fast_exp(x) / e - 1) < 2.5e-4
        assert abs(oracle.fast_exp_fma(x) / e - 1) < 2.5e-4
    assert oracle.fast_exp_fma(0.0) == 1.0 and oracle.fast_exp(0.0) == 1.0
    for x in np.linspace(-80, 0, 200, dtype=np.float32).tolist():
        assert abs(oracle.det_exp(x) / np.exp(np.float64(np.float32(x))) - 1) < 1e-5


def test_paged_attention_blockwise_vs_scalar(oracle):
    """Two reference implementations: blockwise online softmax with the fast-exp polynomial
    (core/src/kernels/hwy/hwy_paged_attention.cc:428-629) and the scalar two-pass one
    (core/src/llm/attention/paged_exec.cpp:37-223); DenseCore's tests hold them to 1e-4-ish."""
    rng = np.random.default_rng(2)
    n_head, n_kv, hd, ctx = 8, 2, 128, 53
    table = np.array([5, 2, 7, 0], np.int32)
    ka = np.zeros((8 * 16, n_kv, hd), np.uint16)
    va = np.zeros_like(ka)
    ks, vs = [], []
    for pos in range(ctx):
        k = rng.normal(size=(n_kv, hd)).astype(np.float32)
        v = rng.normal(size=(n_kv, hd)).astype(np.float32)
        oracle.kv_write(ka, va, table, pos, n_kv, hd, k, v)
        ks.append(k.astype(np.float16).astype(np.float64))
        vs.append(v.astype(np.float16).astype(np.float64))
    # slot layout: block table[pos/16], slot pos%16
    assert ka[5 * 16 + 3, 1, 0] == np.float16(ks[3][1, 0]).view(np.uint16)
    q = rng.normal(size=(n_head, hd)).astype(np.float32)
    scale = 1 / np.sqrt(hd)
    a = oracle.paged_attention(q, ka, va, table, ctx - 1, n_head, n_kv, hd, scale, "blockwise")
    b = oracle.paged_attention(q, ka, va, table, ctx - 1, n_head, n_kv, hd, scale, "scalar")
    Kf, Vf = np.stack(ks), np.stack(vs)
    for h in range(n_head):
        s = (Kf[:, h // 4] @ q[h].astype(np.float64)) * scale
        p = np.exp(s - s.max())
        want = (p[:, None] * Vf[:, h // 4]).sum(0) / p.sum()
        assert np.abs(b[h] - want).max() < 2e-6
        assert np.abs(a[h] - want).max() < 5e-4


def test_rope_rmsnorm_argmax(oracle):
    rng = np.random.default_rng(4)
    x = rng.normal(size=256).astype(np.float32)
    w = rng.normal(size=256).astype(np.float32)
    y = oracle.rms_norm(x, w, 1e-6)
    want = x.astype(np.float64) / np.sqrt((x.astype(np.float64) ** 2).mean() + 1e-6) * w
    assert np.abs(y - want).max() < 1e-5
    tab = oracle.rope_table(32, 128, 1e6)
    pos = 17
    i = np.arange(64)
    ang = pos * (1e6 ** (-2.0 * i / 128))
    assert np.allclose(tab[pos, 0::2], np.cos(ang), atol=1e-6) and np.allclose(tab[pos, 1::2], np.sin(ang), atol=1e-6)
    v = rng.normal(size=(2, 128)).astype(np.float32)
    r = oracle.rope(v, tab[pos])
    want0 = v[:, 0::2] * np.cos(ang) - v[:, 1::2] * np.sin(ang)
    want1 = v[:, 0::2] * np.sin(ang) + v[:, 1::2] * np.cos(ang)
    assert np.allclose(r[:, 0::2], want0, atol=1e-5) and np.allclose(r[:, 1::2], want1, atol=1e-5)
    # first maximum wins (core/src/sampler/sampler.cpp:42-57)
    assert oracle.argmax(np.array([1.0, 5.0, 5.0, 2.0], np.float32)) == 1


def test_verify_accept_rule(oracle):
    rng = np.random.default_rng(8)
    V, gamma = 1000, 4
    tl = (rng.normal(size=(gamma + 1, V)) * 2).astype(np.float32)
    am = [oracle.argmax(r) for r in tl]
    for n_match in range(gamma + 1):
        dt = [am[i] if i < n_match else (am[i] + 1) % V for i in range(gamma)]
        assert oracle.verify_accept(tl, dt, None, None, 0) == (n_match, am[n_match])
    # stochastic: q == p accepts everything (u*q < p for u < 1)
    p = np.stack([oracle.det_softmax(r, 0.8) for r in tl])
    assert np.allclose(p.sum(1), 1.0, atol=1e-5)
    want = np.exp((tl[0] / 0.8).astype(np.float64) - (tl[0] / 0.8).max())
    assert np.allclose(p[0], want / want.sum(), rtol=2e-5, atol=1e-9)
    dt = [int(np.argmax(p[i])) for i in range(gamma)]
    u = oracle.verify_uniforms(1, 0, gamma + 1)
    n, tok = oracle.verify_accept(tl, dt, p[:gamma], u, 1, 0.8)
    assert n == gamma and 0 <= tok < V
    # q puts all mass on a token the target dislikes: rejected at once, resampled elsewhere
    q = np.zeros((gamma, V), np.float32)
    bad = int(np.argmin(p[0]))
    q[:, bad] = 1.0
    n, tok = oracle.verify_accept(tl, [bad] * gamma, q, np.full(gamma + 1, 0.5, np.float32), 1, 0.8)
    assert n == 0 and tok != bad
    # inverse CDF against a float64 restatement
    w = rng.random(5000).astype(np.float32)
    for uu in (0.0, 0.123, 0.5, 0.999):
        i = oracle.det_inverse_cdf(w, uu)
        c = np.cumsum(w.astype(np.float64))
        j = int(np.searchsorted(c, uu * c[-1], side="right"))
        assert abs(i - j) <= 1
    assert oracle.det_inverse_cdf(np.zeros(10, np.float32), 0.3) == -1


def test_synthetic_quantiser_golden_and_quality(oracle):
    assert np.array_equal(oracle.synth_quantized(B.GGML_TYPE_Q4_K, 7, 2, 512, 0.02), GOLD["synth_q4k"])
    assert np.array_equal(oracle.synth_quantized(B.GGML_TYPE_Q6_K, 7, 2, 512, 0.02), GOLD["synth_q6k"])
    src = oracle.synth_normal(7, 0, 1024, 0.02).reshape(2, 512)
    assert abs(src.std() - 0.02) < 0.002 and abs(src.mean()) < 0.003
    e4 = oracle.dequantize(B.GGML_TYPE_Q4_K, GOLD["synth_q4k"], 2, 512) - src
    e6 = oracle.dequantize(B.GGML_TYPE_Q6_K, GOLD["synth_q6k"], 2, 512) - src
    assert e4.std() < 0.1 * src.std() and e6.std() < 0.03 * src.std()


def test_threads_do_not_change_results(oracle):
    rng = np.random.default_rng(9)
    w = B.random_q4k(rng, 64, 512)
    x = rng.normal(size=(2, 512)).astype(np.float32)
    oracle.set_threads(1)
    a = oracle.mul_mat(B.GGML_TYPE_Q4_K, w, 64, 512, x)
    oracle.set_threads(4)
    b = oracle.mul_mat(B.GGML_TYPE_Q4_K, w, 64, 512, x)
    oracle.set_threads(1)
    assert np.array_equal(a, b)
