"""CPU tests of the drop-in boundary: the shared library loads and exports every
symbol the header declares; the host-side mirrors validate their arguments; the
expert-parallel partition arithmetic holds on a 2-rank gloo group."""
import ctypes
import os
import re
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "dc_b200.h")).read()
    return sorted(set(re.findall(r"DC_B200_API[^;(]*?\b(dc_b200_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from densecore_b200 import _lib
    assert os.path.exists(_lib.LIB_PATH), "libdc_b200.so missing: run `python -m densecore_b200.build`"
    lib = ctypes.CDLL(_lib.LIB_PATH)
    declared = header_symbols()
    assert len(declared) >= 50
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/dc_b200.h but not exported"
    # and the Python binding covers exactly the header
    assert sorted(_lib.exported_symbols()) == declared


def test_library_exports_the_ggml_shaped_callbacks():
    """Every entry of include/dc_ggml_compat.h is exported, and the C++ program that drives them builds."""
    from densecore_b200 import _lib
    text = open(os.path.join(ROOT, "include", "dc_ggml_compat.h")).read()
    names = sorted(set(re.findall(r"DC_B200_API[^;(]*?\b(\w+)\s*\(", text)))
    assert names == ["cb_gemv_b200", "cb_moe_forward_b200", "cb_paged_attention_decode_b200", "dc_b200_shim_fail_closed_count"]
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(lib, n), n
    lib.dc_b200_shim_fail_closed_count.restype = ctypes.c_uint64
    assert lib.dc_b200_shim_fail_closed_count() == 0
    # a callback entered by a thread other than 0 returns at once, whatever it is given
    lib.cb_gemv_b200(None, 1, 4, None)
    lib.cb_moe_forward_b200(None, None, None, 3, 4, None)
    lib.cb_paged_attention_decode_b200(None, 2, 4, None)
    # thread 0 with no result tensor has nothing to fill and nothing to count
    lib.cb_gemv_b200(None, 0, 4, None)
    assert lib.dc_b200_shim_fail_closed_count() == 0
    from oracle import oracle as o
    o.build()
    subprocess.check_call(["make", "-C", os.path.join(ROOT, "tests", "shims"), "ggml_shims_test"], stdout=subprocess.DEVNULL)
    assert os.path.exists(os.path.join(ROOT, "tests", "shims", "ggml_shims_test"))


def test_prefix_cache_key_is_the_reference_hash():
    """The prefix cache keys a block by FNV-1a over the token ids of the whole prefix, one 64-bit step per id
    (BlockManager::ComputeTokenHash, core/src/runtime/memory/kv_cache_block_manager.cpp:515-522, salt 0): checked
    against a Python restatement, including the known FNV-1a offset basis for an empty continuation."""
    from densecore_b200 import _lib
    lib = _lib.lib()

    def ref(tokens):
        h = 14695981039346656037
        for t in tokens:
            h ^= int(t) & 0xFFFFFFFFFFFFFFFF
            h = (h * 1099511628211) & 0xFFFFFFFFFFFFFFFF
        return h

    rng = np.random.default_rng(0)
    for n in (1, 15, 16, 17, 1024):
        toks = rng.integers(0, 151936, size=n).astype(np.int32)
        assert lib.dc_b200_kv_prefix_hash(toks.ctypes.data_as(ctypes.c_void_p), n) == ref(toks), n
    one = np.array([0], dtype=np.int32)
    assert lib.dc_b200_kv_prefix_hash(one.ctypes.data_as(ctypes.c_void_p), 1) == (14695981039346656037 * 1099511628211) % 2 ** 64
    # a different left context changes the key of the same block contents
    a = np.arange(32, dtype=np.int32)
    b = a.copy()
    b[0] = 99
    assert lib.dc_b200_kv_prefix_hash(a.ctypes.data_as(ctypes.c_void_p), 32) != lib.dc_b200_kv_prefix_hash(b.ctypes.data_as(ctypes.c_void_p), 32)
    assert lib.dc_b200_kv_prefix_hash(None, 0) == 0


def test_no_cpu_fallback_without_gpu():
    """On a machine without a GPU, init fails loudly instead of computing on the CPU."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import densecore_b200 as dc
    with pytest.raises(dc.DcError) as e:
        dc.Context(0)
    assert e.value.status == -6


def test_product_never_imports_the_oracle():
    """The shipped package neither imports, loads nor links anything under oracle/."""
    pat = re.compile(r"import\s+oracle|from\s+oracle|from\s+\.+oracle|libdc_oracle|oracle/|dco_\w+")
    for dirpath, _, files in os.walk(os.path.join(ROOT, "densecore_b200")):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert not pat.search(text), f"{f} refers to the oracle"
    out = subprocess.run(["ldd", os.path.join(ROOT, "densecore_b200", "libdc_b200.so")], capture_output=True, text=True)
    assert "oracle" not in out.stdout


def test_block_generators_shapes_and_ranges():
    from densecore_b200 import blocks as B
    rng = np.random.default_rng(0)
    w4 = B.random_q4k(rng, 3, 512)
    w6 = B.random_q6k(rng, 3, 512)
    assert w4.shape == (3, 288) and w6.shape == (3, 420)
    assert B.row_bytes(B.GGML_TYPE_Q4_K, 2048) == 1152 and B.row_bytes(B.GGML_TYPE_Q6_K, 2048) == 1680
    with pytest.raises(ValueError):
        B.row_bytes(B.GGML_TYPE_Q4_K, 100)
    sc = w6.reshape(3, 2, 210)[:, :, 192:208].view(np.int8)
    assert sc.min() >= -32 and sc.max() <= 31


def test_model_config_mirrors_c_struct():
    import densecore_b200 as dc
    from densecore_b200 import _lib
    c = dc.moe_35b_a3b().to_c()
    assert (c.n_layer, c.hidden, c.n_head, c.n_kv_head, c.n_expert, c.n_expert_used, c.expert_ffn, c.vocab) == \
        (48, 2048, 32, 4, 128, 8, 768, 151936)
    d = dc.dense_0p8b().to_c()
    assert (d.n_layer, d.hidden, d.ffn, d.n_head, d.n_kv_head, d.tie_embeddings) == (28, 1024, 3072, 16, 8, 1)
    assert ctypes.sizeof(_lib.ModelConfig) == 19 * 4
    assert dc.tensor_seed(5, "blk.0.attn_q.weight") == (5 + dc.model.fnv1a64("blk.0.attn_q.weight")) % 2 ** 64


EP_WORKER = r'''
import os, sys
import numpy as np
import torch
import torch.distributed as dist
sys.path.insert(0, os.environ["DC_ROOT"])
from oracle import oracle as o
from densecore_b200 import blocks as B
dist.init_process_group("gloo", rank=int(os.environ["RANK"]), world_size=int(os.environ["WORLD_SIZE"]))
rank, world = dist.get_rank(), dist.get_world_size()
rng = np.random.default_rng(21)          # same seed on every rank: replicated router and inputs
H, F, E, K, T = 512, 256, 8, 2, 3
gate, up = B.random_q4k(rng, E * F, H), B.random_q4k(rng, E * F, H)
down = B.random_q6k(rng, E * H, F)
x = rng.normal(size=(T, H)).astype(np.float32)
ids, w = o.route(rng.normal(size=(T, E)).astype(np.float32), K)
types = (12, 12, 14)
full = o.moe_forward(types, gate, up, down, E, H, F, x, ids, w)
# this rank owns experts [lo, hi): weights of assignments to other ranks' experts are zeroed,
# which is what "skip non-local assignments" means; partial outputs are summed by all-reduce
per = E // world
lo, hi = rank * per, (rank + 1) * per
w_local = np.where((ids >= lo) & (ids < hi), w, 0.0).astype(np.float32)
part = torch.from_numpy(o.moe_forward(types, gate, up, down, E, H, F, x, ids, w_local))
dist.all_reduce(part)
err = float(np.abs(part.numpy() - full).max() / np.abs(full).max())
assert err < 1e-5, err
if rank == 0:
    print("EP_OK", err)
dist.destroy_process_group()
'''


def test_expert_parallel_partition_sums_to_full_layer_gloo(tmp_path):
    """World size 2 on CPU (gloo): per-rank expert shards + one sum all-reduce reproduce the full layer."""
    script = tmp_path / "ep_worker.py"
    script.write_text(EP_WORKER)
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT="29731",
                   DC_ROOT=ROOT)
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=180)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)
    assert "EP_OK" in outs[0]
