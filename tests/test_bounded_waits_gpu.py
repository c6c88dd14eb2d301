"""Bounded waits of the persistent decode kernel: a wait that runs out comes back as a status, the kernel
leaves cleanly (no computing on unsynchronised data, copies in flight drained), and the context stays usable.
The failure is made by shortening the limit (a barrier poll budget of one; a peer that nothing ever signals),
never by faulting, trapping or hanging the GPU."""
import numpy as np
import pytest

import densecore_b200 as dc

pytestmark = pytest.mark.gpu

CFG = dict(n_layer=2, hidden=512, n_head=4, n_kv_head=2, vocab=1000, n_expert=8, n_expert_used=2, expert_ffn=256,
           max_seqs=2, max_ctx=128)


def test_grid_barrier_poll_limit_runs_out_and_the_next_call_works(ctx):
    m = dc.Model(ctx, dc.Config(**CFG))
    m.init_synthetic(7, 0.05)
    m.finalize()
    m.set_option("persistent", 2)
    s = m.seq_alloc()
    first = m.prefill(s, np.arange(20) % 1000)
    want, _ = m.decode_run([s], [first], 6)
    assert m.step_stats()[0] == 1                       # the persistent kernel ran
    m.seq_truncate(s, 20)
    # one poll per barrier: some CTA of 148 finds the others not there yet, gives up, and the launch ends
    m.set_option("test_barrier_polls", 1)
    with pytest.raises(dc.DcError) as e:
        m.decode_run([s], [first], 6)
    assert e.value.status == -6 and "bounded wait" in str(e.value) and "code 2" in str(e.value)
    # the default limit again: the same steps give the same tokens (the failed run left no state behind that
    # the retry does not overwrite)
    m.set_option("test_barrier_polls", 0)
    m.seq_truncate(s, 20)
    again, _ = m.decode_run([s], [first], 6)
    assert np.array_equal(again, want)
    m.close()


def test_expert_parallel_wait_runs_out_on_a_peer_that_never_arrives(ctx):
    cfg = dc.Config(ep_rank=0, ep_size=2, **CFG)
    m = dc.Model(ctx, cfg)
    m.init_synthetic(7, 0.05)
    m.set_option("test_ep_loopback", 1)                 # the peer's buffer is local and nothing signals it
    m.finalize()
    m.set_option("persistent", 2)
    m.set_option("test_ep_wait_us", 1000)               # one millisecond instead of two seconds
    s = m.seq_alloc()
    with pytest.raises(dc.DcError) as e:
        m.decode_run([s], [5], 3)
    assert e.value.status == -6 and "code 3" in str(e.value)
    m.close()
    # the context is still good for other work
    from densecore_b200 import blocks as B
    rng = np.random.default_rng(0)
    w = B.random_q4k(rng, 64, 256)
    W = ctx.upload_weight(B.GGML_TYPE_Q4_K, w, 256, 64)
    y = ctx.mul_mat(W, rng.normal(size=(1, 256)).astype(np.float32))
    assert np.isfinite(y).all()
    W.free()
