"""One rank of the 2-GPU expert-parallel check (run by tests/test_ep_gpu.py under torch.distributed.run).

Every rank builds its shard of a cut-down MoE decoder; rank 0 also builds the whole model on its own GPU.
Greedy tokens of the sharded runs (peer-store exchange inside the persistent kernel, and the per-op path
with an NCCL all-reduce) are compared with the single-GPU tokens."""
import ctypes as C
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import densecore_b200 as dc  # noqa: E402


def main():
    rank, world, lr = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.cuda.set_device(lr)
    ctx = dc.Context(lr)

    def make(ep_rank, ep_size, peer):
        cfg = dc.moe_35b_a3b(max_seqs=4, max_ctx=512, ep_rank=ep_rank, ep_size=ep_size)
        cfg.n_layer, cfg.vocab = 3, 8192
        m = dc.Model(ctx, cfg)
        m.init_synthetic(1234, 0.02)
        if ep_size > 1:
            import nvidia.nccl
            nccl_path = os.path.join(list(nvidia.nccl.__path__)[0], "lib", "libnccl.so.2")
            buf = torch.zeros(128, dtype=torch.uint8)
            if rank == 0:
                raw = (C.c_char * 128)()
                ctx._check(dc._lib.lib().dc_b200_ep_unique_id(ctx.handle, nccl_path.encode(), raw))
                buf = torch.frombuffer(bytearray(raw.raw), dtype=torch.uint8).clone()
            dist.broadcast(buf, 0)
            m.ep_init(bytes(buf.numpy().tobytes()), nccl_path)
            if peer:
                mine = torch.frombuffer(bytearray(m.ep_export()), dtype=torch.uint8).clone()
                handles = [torch.zeros(64, dtype=torch.uint8) for _ in range(world)]
                dist.all_gather(handles, mine)
                for r in range(world):
                    if r != rank:
                        m.ep_import(r, bytes(handles[r].numpy().tobytes()))
        m.finalize()
        m.set_option("persistent", 2 if peer or ep_size == 1 else 0)
        # bit-identity across GPU counts: every model prefills through the same (sixteen-token) path
        m.set_option("tc_prefill", 0)
        return m

    def run(m):
        rng = np.random.default_rng(0)
        out = {}
        # (a) sequences that start empty: every token goes through the decode path under test, nothing through
        # the chunked prefill (whose expert sum is an all-reduce in a different order)
        for T in (1, 4):
            seqs = [m.seq_alloc() for _ in range(T)]
            start = rng.integers(0, 8192, size=T)
            toks, _ = m.decode_run(seqs, start, 24)
            last, lg = m.decode_step(seqs, toks[-1], want_logits=True)
            out[("fresh", T)] = (toks, last, m.step_stats()[0], lg.copy())
            for s in seqs:
                m.seq_free(s)
        # (b) after prompts
        prompts = [rng.integers(0, 8192, size=150 + 7 * i) for i in range(4)]
        seqs = [m.seq_alloc() for _ in range(4)]
        first = [m.prefill(s, p) for s, p in zip(seqs, prompts)]
        for T in (1, 4):
            toks, _ = m.decode_run(seqs[:T], first[:T], 12)
            last = m.decode_step(seqs[:T], toks[-1])
            out[("prompt", T)] = (toks, last, m.step_stats()[0], None)
        for s in seqs:
            m.seq_free(s)
        # (c) prompts through the tensor-core chunked prefill (local experts' GEMMs, one all-reduce per layer)
        m.set_option("tc_prefill", 1)
        s = m.seq_alloc()
        first = m.prefill(s, prompts[3])
        toks, _ = m.decode_run([s], [first], 12)
        out[("tc", 1)] = (np.concatenate([[[first]], toks]), None, 0, None)
        m.seq_free(s)
        m.set_option("tc_prefill", 0)
        return out

    res = {}
    for name, peer in (("peer", True), ("nccl", False)):
        m = make(rank, world, peer)
        dist.barrier()
        res[name] = run(m)
        dist.barrier()      # every rank is done with its peers' buffers before any rank frees its own
        m.close()
        dist.barrier()
    ok = True
    if rank == 0:
        ref = make(0, 1, False)
        want = run(ref)
        ref.close()
        for T in (1, 4):
            peer, nccl, one = res["peer"][("fresh", T)], res["nccl"][("fresh", T)], want[("fresh", T)]
            same_peer = np.array_equal(peer[0], one[0]) and np.array_equal(peer[1], one[1]) and np.array_equal(peer[3], one[3])
            agree_nccl = float((nccl[0] == one[0]).mean())
            print(f"T={T}, fresh sequences: peer exchange identical to one GPU (tokens and logits): {same_peer} "
                  f"(launches/step {peer[2]}); NCCL path token agreement {agree_nccl:.3f} (launches/step {nccl[2]})")
            ok &= same_peer and peer[2] == 1 and nccl[2] > 1 and agree_nccl > 0.7
            peer, nccl, one = res["peer"][("prompt", T)], res["nccl"][("prompt", T)], want[("prompt", T)]
            a_peer, a_nccl = float((peer[0] == one[0]).mean()), float((nccl[0] == one[0]).mean())
            print(f"T={T}, after prompts (prefill sums experts by all-reduce): token agreement peer {a_peer:.3f}, NCCL {a_nccl:.3f}")
            ok &= a_peer > 0.6 and a_nccl > 0.6
        for name in ("peer", "nccl"):
            a = float((res[name][("tc", 1)][0] == want[("tc", 1)][0]).mean())
            print(f"tensor-core prefill on two GPUs ({name} model): token agreement with one GPU {a:.3f}")
            ok &= a > 0.6
        print("EP OK" if ok else "EP MISMATCH")
    dist.barrier()
    dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
