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
        return m

    def run(m):
        rng = np.random.default_rng(0)
        prompts = [rng.integers(0, 8192, size=150 + 7 * i) for i in range(4)]
        seqs = [m.seq_alloc() for _ in range(4)]
        first = [m.prefill(s, p) for s, p in zip(seqs, prompts)]
        out = {}
        for T in (1, 4):
            toks, _ = m.decode_run(seqs[:T], first[:T], 12)
            last = m.decode_step(seqs[:T], toks[-1])
            out[T] = (toks, last, m.step_stats()[0])
        return out

    res = {}
    for name, peer in (("peer", True), ("nccl", False)):
        m = make(rank, world, peer)
        dist.barrier()
        res[name] = run(m)
        m.close()
        dist.barrier()
    ok = True
    if rank == 0:
        ref = make(0, 1, False)
        want = run(ref)
        ref.close()
        for T in (1, 4):
            peer, nccl = res["peer"][T], res["nccl"][T]
            same_peer = np.array_equal(peer[0], want[T][0]) and np.array_equal(peer[1], want[T][1])
            agree_nccl = float((nccl[0] == want[T][0]).mean())
            print(f"T={T}: peer exchange identical to one GPU: {same_peer} (launches/step {peer[2]}); "
                  f"NCCL path token agreement {agree_nccl:.3f} (launches/step {nccl[2]})")
            ok &= same_peer and peer[2] == 1 and nccl[2] > 1 and agree_nccl > 0.8
        print("EP OK" if ok else "EP MISMATCH")
    dist.barrier()
    dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
