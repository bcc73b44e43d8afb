"""Expert-parallel MoE layers: the exchange of contribution rows between ranks.

One GPU: the delivery code runs against stand-in peers that never answer, so the bounded wait
runs out and the call reports it (the failure is made by a flag that nothing sets; no fault, no
hang). Two GPUs (skipped when the box has one): two processes, one engine each, own halves of the
experts, exchange over peer mappings, results against the one-GPU CPU path.
"""
import os

import numpy as np
import pytest

import common
import synth

pkg = synth.pkg
pytestmark = pytest.mark.gpu


def _tiny():
    spec = synth.tiny_spec()
    return spec, synth.make_model(spec, seed=11, recipe="baseline")


def test_unanswered_exchange_times_out_and_is_reported(gpu_lib, binding):
    spec, tensors = _tiny()
    eng = pkg.Engine(spec.cfg, spec.is_mla, spec.is_dense, 32, 0, 0, 2)     # rank 0 of 2
    eng.load_all(tensors); eng.finalize()
    moe_layer = next(l for l in range(spec.cfg.n_layers) if not spec.is_dense[l])
    x = synth.moe_inputs(spec.cfg, 2, 3)
    with pytest.raises(RuntimeError, match="connect the ranks"):
        eng.op_moe(moe_layer, x)
    eng.set_option("ep_loopback", 1)
    eng.set_option("ep_wait_ms", 300)                  # the stand-in peers never answer: do not wait 5 s for them
    with pytest.raises(RuntimeError, match="timed out"):
        eng.op_moe(moe_layer, x)
    # a failed step poisons the step count; resync restarts it, and the next step fails the same clean way
    eng.ep_resync()
    with pytest.raises(RuntimeError, match="timed out"):
        eng.op_moe(moe_layer, x[:1])
    # a forward pass that fails half-way leaves the session undefined: refused until reset
    eng.ep_resync()
    ids = [1, 2, 3]
    with pytest.raises(RuntimeError, match="timed out"):
        eng.forward(ids)
    with pytest.raises(RuntimeError, match="reset the engine"):
        eng.forward(ids)
    eng.reset()
    assert eng.cached == 0
    eng.close()
    # the context is still usable: a one-GPU engine on the same device gives the CPU path's output
    one, orc = common.build_models(spec, tensors, 32, binding)
    assert common.rel_err(one.op_moe(moe_layer, x), orc.op_moe(moe_layer, x)) < 1e-5
    one.close(); orc.close()


def _rank_main(rank, world, conn, peers_conn):
    """Child process: one rank of an expert-parallel pair. Results go back through `conn`."""
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, os.path.dirname(here)); sys.path.insert(0, here)
    import numpy as np
    import synth as sy
    import common as cm
    from oracle import binding
    try:
        spec = sy.tiny_spec()
        tensors = sy.make_model(spec, seed=11, recipe="baseline")
        eng = sy.pkg.Engine(spec.cfg, spec.is_mla, spec.is_dense, 32, rank, rank, world)
        eng.load_all(tensors); eng.finalize()
        conn.send(("handle", eng.ep_export()))
        handles = conn.recv()
        eng.ep_connect(handles)
        orc = binding.OracleModel(spec.cfg, spec.is_mla, spec.is_dense, 32, 2)
        orc.load_all(tensors); orc.finalize()
        moe_layer = next(l for l in range(spec.cfg.n_layers) if not spec.is_dense[l])
        worst = 0.0
        for T, seed in ((1, 1), (4, 2), (1, 3), (7, 4), (32, 5)):
            x = sy.moe_inputs(spec.cfg, T, seed)
            worst = max(worst, cm.rel_err(eng.op_moe(moe_layer, x), orc.op_moe(moe_layer, x)))
        ids = np.random.default_rng(0).integers(0, spec.cfg.vocab, 18).tolist()
        lg, _ = eng.forward(ids)
        lw, _ = orc.forward(ids)
        fw = cm.rel_err(lg, lw)
        steps = []
        for _ in range(4):
            tok = int(np.argmax(lg)); assert tok == int(np.argmax(lw))
            lg, _ = eng.forward([tok]); lw, _ = orc.forward([tok])
            steps.append(cm.rel_err(lg, lw))
        # greedy decode on the device: the head is split by vocabulary rows, the ranks exchange their
        # (value, index) pairs; the tokens must be the CPU path's
        tok = int(np.argmax(lw))
        got = eng.decode_greedy(tok, 5)
        want = []
        for _ in range(5):
            lw, _ = orc.forward([tok])
            tok = int(np.argmax(lw)); want.append(tok)
        assert got.tolist() == want, (got.tolist(), want)
        eng.close(); orc.close()
        # the full-size layer: 144 routed experts per rank; batch 1 takes the tensor-core kernels,
        # larger batches the register kernels, both end in the exchange
        spec = sy.layer_spec("moe")
        trunk = sy.moe_layer_trunk(spec, 0)
        big = sy.pkg.Engine(spec.cfg, spec.is_mla, spec.is_dense, 8, rank, rank, world)
        big.set_option("allow_partial", 1)
        big.load_all(trunk)
        for ex in range(spec.cfg.n_experts):
            big.fill_expert(0, ex, 0, *sy.expert_scales(spec.cfg, 0, ex, 0))
        big.finalize()
        conn.send(("handle", big.ep_export()))
        big.ep_connect(conn.recv())
        full = 0.0
        for T, seed in ((1, 7), (1, 8), (8, 9)):
            x = sy.moe_inputs(spec.cfg, T, seed)
            idx, _ = big.op_router(0, x)
            ref = sy.oracle_moe_layer(binding, spec, trunk, 0, idx.ravel())
            full = max(full, cm.rel_err(big.op_moe(0, x), ref.op_moe(0, x)))
            ref.close()
        big.close()
        # speculative greedy decode on the MTP layer's drafts across the ranks (heads split, so each rank
        # keeps and restores only its own heads' KDA state): the tokens of plain greedy decode on the CPU
        spec = sy.tiny_spec()
        spec.cfg.vocab = 4                                     # a draft is right often enough for both outcomes
        tensors = sy.make_model(spec, seed=9, recipe="spread")
        tensors.update(sy.make_mtp_layer(spec, seed=9, recipe="spread"))
        eng = sy.pkg.Engine(spec.cfg, spec.is_mla, spec.is_dense, 64, rank, rank, world)
        eng.enable_mtp()
        eng.load_all(tensors); eng.finalize()
        conn.send(("handle", eng.ep_export()))
        eng.ep_connect(conn.recv())
        orc = binding.OracleModel(spec.cfg, spec.is_mla, spec.is_dense, 64, 2)
        orc.load_all({k: v for k, v in tensors.items() if not k.startswith(f"layers.{spec.cfg.n_layers}.")}); orc.finalize()
        prompt = np.random.default_rng(3).integers(0, 4, 9).astype(np.int32)
        lg, _ = eng.forward(prompt); lw, _ = orc.forward(prompt)
        tok = int(np.argmax(lw)); assert int(np.argmax(lg)) == tok
        hid = eng.mtp_hidden(0, prompt.size)
        eng.mtp_feed(prompt[1:], hid[:-1], want_draft=False)
        got, stats = eng.decode_speculative(tok, 20)
        want = []
        for _ in range(20):
            lw, _ = orc.forward([tok])
            tok = int(np.argmax(lw)); want.append(tok)
        assert got.tolist() == want, (got.tolist(), want)
        assert 0 < stats["accepted"] < stats["drafts"], stats
        eng.close(); orc.close()
        conn.send(("ok", worst, fw, max(steps), full))
    except Exception as exc:                                   # report instead of dying silently
        conn.send(("error", repr(exc)))


def _seq_rank_main(rank, world, conn, peers_conn):
    """Child process: one rank of a pair that splits the SEQUENCES. Every rank runs attention and all
    other per-token work for its own two sequences; MoE layers gather the ranks' tokens, each rank
    multiplies them by the experts it owns and sends the rows to the token's rank."""
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, os.path.dirname(here)); sys.path.insert(0, here)
    import numpy as np
    import synth as sy
    import common as cm
    from oracle import binding
    try:
        spec = sy.tiny_spec()
        tensors = sy.make_model(spec, seed=31, recipe="spread")
        S, cap, plen, steps = 2, 40, 17, 6
        eng = sy.pkg.Engine(spec.cfg, spec.is_mla, spec.is_dense, cap, rank, rank, world)
        eng.set_option("sequences", S)
        eng.set_option("sequence_split", 1)
        eng.load_all(tensors); eng.finalize()
        conn.send(("handle", eng.ep_export()))
        eng.ep_connect(conn.recv())
        rng = np.random.default_rng(50 + rank)                    # every rank has its own prompts
        prompts = [rng.integers(0, spec.cfg.vocab, plen).tolist() for _ in range(S)]
        orcs, last, worst = [], [], 0.0
        for q in range(S):
            o = binding.OracleModel(spec.cfg, spec.is_mla, spec.is_dense, cap, 2)
            o.load_all(tensors); o.finalize()
            orcs.append(o)
            eng.use_sequence(q)
            lg, _ = eng.forward(prompts[q])
            lw, _ = o.forward(prompts[q])
            worst = max(worst, cm.rel_err(lg, lw))
            last.append(int(np.argmax(lw)))
        same = True
        for step in range(steps):
            lg, am = eng.decode_batch(last)
            nxt = []
            for q in range(S):
                lw, _ = orcs[q].forward([last[q]])
                worst = max(worst, cm.rel_err(lg[q], lw))
                same = same and int(am[q]) == int(np.argmax(lw))
                nxt.append(int(np.argmax(lw)))
            last = nxt
        moe_layer = next(l for l in range(spec.cfg.n_layers) if not spec.is_dense[l])
        op = 0.0
        for T, seed in ((1, 1), (5, 2), (64, 3)):                 # 64 per rank: two groups of gathered tokens
            x = sy.moe_inputs(spec.cfg, T, seed + 10 * rank)
            op = max(op, cm.rel_err(eng.op_moe(moe_layer, x), orcs[0].op_moe(moe_layer, x)))
        eng.close()
        for o in orcs:
            o.close()
        # the full-size layer, 144 experts per rank, own tokens per rank
        spec = sy.layer_spec("moe")
        trunk = sy.moe_layer_trunk(spec, 0)
        big = sy.pkg.Engine(spec.cfg, spec.is_mla, spec.is_dense, 8, rank, rank, world)
        big.set_option("allow_partial", 1)
        big.set_option("sequence_split", 1)
        big.load_all(trunk)
        for ex in range(spec.cfg.n_experts):
            big.fill_expert(0, ex, 0, *sy.expert_scales(spec.cfg, 0, ex, 0))
        big.finalize()
        conn.send(("handle", big.ep_export()))
        big.ep_connect(conn.recv())
        full = 0.0
        for T, seed in ((1, 7), (8, 8), (32, 9)):
            x = sy.moe_inputs(spec.cfg, T, seed + 10 * rank)
            idx, _ = big.op_router(0, x)
            ref = sy.oracle_moe_layer(binding, spec, trunk, 0, idx.ravel())
            full = max(full, cm.rel_err(big.op_moe(0, x), ref.op_moe(0, x)))
            ref.close()
        big.close()
        conn.send(("ok", worst, 0.0 if same else 1.0, op, full))
    except Exception as exc:
        conn.send(("error", repr(exc)))


def _mla_rank_main(rank, world, conn, peers_conn):
    """Child process: full-size MLA layers split by heads over two ranks, BF16 latent cache (the
    tensor-core attention core). 64 heads: 32 per rank. 16 heads: 8 per rank, fewer than the core's
    group of 16 - one new token pads the group with zero queries, several positions keep the layer
    whole. Caches seeded directly; every output against the CPU path."""
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, os.path.dirname(here)); sys.path.insert(0, here)
    import numpy as np
    import synth as sy
    import common as cm
    from oracle import binding
    try:
        worst = []
        for heads in (64, 16):
            spec = sy.layer_spec("mla")
            c = spec.cfg
            c.mla_heads = heads
            cap = 8192
            tensors = sy.make_model(spec, seed=5, recipe="spread")
            eng = sy.pkg.Engine(c, spec.is_mla, spec.is_dense, cap, rank, rank, world)
            eng.set_option("allow_partial", 1)
            eng.set_option("latent_bf16", 1)
            eng.load_all(tensors); eng.finalize()
            conn.send(("handle", eng.ep_export()))
            eng.ep_connect(conn.recv())
            orc = binding.OracleModel(c, spec.is_mla, spec.is_dense, cap, 2)
            orc.load_all(tensors); orc.finalize()
            rng = np.random.default_rng(5)
            lat = sy.bf16_round(rng.standard_normal((cap, c.kv_lora)).astype(np.float32))
            idx = rng.standard_normal(2 * cap * c.index_dim + (cap // c.index_kpool) * c.index_dim).astype(np.float32)
            for m in (eng, orc):
                m.state_write(0, 1, 0, lat)
                m.state_write(0, 2, 0, idx)
            w = 0.0
            for ctx, T in ((2048, 1), (8000, 1), (8000, 5)):
                x = sy.bf16_round(rng.standard_normal((T, c.hidden)).astype(np.float32))
                (g, gs), (o, os_) = eng.op_mla(0, x, ctx - T), orc.op_mla(0, x, ctx - T)
                assert (gs is None and os_ is None) or np.array_equal(gs, os_), (heads, ctx, T)
                w = max(w, cm.rel_err(g, o))
            worst.append(w)
            eng.close(); orc.close()
        conn.send(("ok", worst[0], worst[1]))
    except Exception as exc:
        conn.send(("error", repr(exc)))


def _run_pair(target, bars, rounds=2):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import multiprocessing as mp
    ctx = mp.get_context("spawn")
    world = 2
    pipes = [ctx.Pipe() for _ in range(world)]
    procs = [ctx.Process(target=target, args=(r, world, pipes[r][1], None)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        for _ in range(rounds):                             # one exchange of handles per engine the ranks build
            handles = []
            for r in range(world):
                assert pipes[r][0].poll(600), "rank did not export its handle"
                msg = pipes[r][0].recv()
                assert msg[0] == "handle", msg
                handles.append(msg[1])
            for r in range(world):
                pipes[r][0].send(handles)
        for r in range(world):
            assert pipes[r][0].poll(600), "rank did not finish"
            msg = pipes[r][0].recv()
            assert msg[0] == "ok", msg
            assert all(v < bar for v, bar in zip(msg[1:], bars)), msg
    finally:
        for p in procs:
            p.join(timeout=60)
            if p.is_alive():
                p.kill()


def test_two_ranks_split_the_sequences_and_match_the_cpu_path(gpu_lib):
    """Logits of every rank's own sequences within 1e-3 of separate CPU sessions with identical
    arg-max, MoE ops on own tokens (one group and two groups of gathered tokens) within 1e-5."""
    _run_pair(_seq_rank_main, (1e-3, 0.5, 1e-5, 1e-5))


def test_two_ranks_split_the_mla_heads(gpu_lib):
    """Within the BF16 latent cache's 3e-3 of the CPU path (which keeps FP32 latents), selections identical."""
    _run_pair(_mla_rank_main, (3e-3, 3e-3), rounds=2)


def test_two_ranks_exchange_and_match_the_cpu_path(gpu_lib):
    _run_pair(_rank_main, (1e-5, 1e-3, 1e-3, 1e-5), rounds=3)
