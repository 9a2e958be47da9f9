"""The producer (forward pass), the round loop and the generation loops on the GPU against the CPU oracle,
on the CPU-runnable tiny configuration: 4-layer Llama-style target, draft = its first 2 layers + shared head."""
import numpy as np
import pytest

from tests import weights

pytestmark = pytest.mark.gpu
REL, ABS = 2e-3, 1e-3


@pytest.fixture(scope="module")
def rig(oracle):
    import turbospark_b200 as tsb
    ctx = tsb.Ctx(0)
    cfg = tsb.config_tiny(max_context=512)
    dcfg = tsb.ModelConfig(2, cfg.d_model, cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim, cfg.ffn, cfg.vocab, cfg.max_context,
                           cfg.rms_eps, cfg.rope_theta)
    mats, norms = weights.random_weights(cfg, 0, oracle, real_ffn=1408)
    target = tsb.Model(ctx, cfg)
    weights.load_weights(target, mats, norms)
    draft = tsb.Model(ctx, dcfg)
    for l in range(2):
        draft.share(l, target, l)
    draft.share(-1, target, -1)
    # the oracle's copies
    ocfg = oracle.ModelCfg(cfg.n_layers, cfg.d_model, cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim, cfg.ffn, cfg.vocab,
                           cfg.max_context, cfg.rms_eps, cfg.rope_theta)
    odcfg = oracle.ModelCfg(2, cfg.d_model, cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim, cfg.ffn, cfg.vocab, cfg.max_context,
                            cfg.rms_eps, cfg.rope_theta)
    ot = oracle.Model(ocfg, threads=8)
    weights.load_weights(ot, mats, norms)
    od = oracle.Model(odcfg, threads=8)
    weights.load_weights(od, mats, norms, layers=2)
    yield dict(ctx=ctx, cfg=cfg, target=target, draft=draft, ot=ot, od=od, tsb=tsb)
    target.close(), draft.close(), ctx.close()


def _close(oracle, got16, want16, rel=REL, abs_=ABS):
    got, want = oracle.f16_bits_to_f32(got16), oracle.f16_bits_to_f32(want16)
    assert not np.isnan(got).any()
    err = np.abs(got - want)
    assert np.all(err <= abs_ + rel * np.abs(want)), float(err.max())


def test_decode_and_verify_logits_match_the_oracle_forward(rig, oracle):
    tsb = rig["tsb"]
    sess = tsb.Session(rig["ctx"], rig["target"], rig["draft"], 1, 8)
    ost = oracle.State(rig["ot"])
    rng = np.random.default_rng(1)
    prompt = rng.integers(0, rig["cfg"].vocab, size=12).astype(np.int32)
    # token-by-token decode
    for i, t in enumerate(prompt):
        got = sess.produce(int(t), i)
        want = ost.forward([int(t)], i)[0]
        _close(oracle, got, want, rel=4e-3, abs_=4e-3)  # f16 rounding points compound over 4 layers
    # a 6-row verify at the cursor must equal decoding the same rows one by one, bit for bit
    feed = rng.integers(0, rig["cfg"].vocab, size=6).astype(np.int32)
    point = sess.checkpoint()
    batch = sess.verify(feed, point)
    sess.rollback_retaining(point, 0)
    single = np.stack([sess.produce(int(t), point + i) for i, t in enumerate(feed)])
    assert np.array_equal(batch, single)
    want = ost.forward(feed, point)
    _close(oracle, batch, want, rel=4e-3, abs_=4e-3)
    # the cursor contract: a position that does not continue the cache is refused and changes nothing
    with pytest.raises(tsb.TsbError):
        sess.produce(1, point)
    assert sess.checkpoint() == point + 6
    sess.close()


def test_tree_verify_matches_the_oracle_and_compaction_restores_a_chain(rig, oracle):
    tsb = rig["tsb"]
    sess = tsb.Session(rig["ctx"], rig["target"], rig["draft"], 1, 8)
    ost = oracle.State(rig["ot"])
    rng = np.random.default_rng(2)
    prompt = rng.integers(0, rig["cfg"].vocab, size=20).astype(np.int32)
    for i, t in enumerate(prompt):
        sess.produce_prefill(int(t), i)
    ost.forward(prompt, 0, want_logits=False)
    parent = [-1, 0, 1, 2, 3, 0, 5, 2]
    feed = rng.integers(0, rig["cfg"].vocab, size=8).astype(np.int32)
    base = sess.checkpoint()
    got = sess.verify_tree(feed, parent, base)
    want = ost.forward(feed, base, parent=parent)
    _close(oracle, got, want, rel=4e-3, abs_=4e-3)
    # accept the branch 0 -> 5 -> 6: the reference's own sequence (crates/runtime/src/speculative.rs:530-567) compacts
    # the path to rows 0..2, cuts the verify back to them, closes the round and records what was kept
    sess.compact_tree(base, [0, 5, 6])
    sess.rollback_retaining(base, 3)
    sess.commit_pending(3)
    kept = [int(feed[0]), int(feed[5]), int(feed[6])]
    sess.record_committed(kept, base)
    sess.rewind_drafter(base + 2)
    assert sess.checkpoint() == base + 3
    ost.cursor = base
    ost.forward(kept, base)
    # the drafter replays the record of fed tokens: its next step must see the path's tokens, not zeros
    odst = oracle.State(rig["od"])
    odst.forward(list(prompt) + kept, 0, want_logits=False)
    nxt = 77
    _close(oracle, sess.draft_step(nxt, base + 2), odst.forward([nxt], base + 3)[0], rel=4e-3, abs_=4e-3)
    _close(oracle, sess.produce(nxt, base + 3), ost.forward([nxt], base + 3)[0], rel=4e-3, abs_=4e-3)
    # and a later turn finds the kept rows under the tokens that were really fed
    assert sess.try_reuse_prefix(list(prompt) + kept + [nxt, 5]) == len(prompt) + 4
    # a second compaction of the same verify, and keeping rows nobody recorded, are refused
    with pytest.raises(tsb.TsbError):
        sess.compact_tree(base, [0, 5, 6])
    sess.close()


@pytest.mark.parametrize("streams", [3, 5])
def test_a_tree_verify_over_every_stream_in_one_pass_equals_the_per_stream_calls(rig, oracle, streams):
    """3 streams x 7 slots stay on the few-row matmul path, 5 x 7 = 35 rows take the many-row one; in both the
    batched pass gives each stream the bits its own verify_tree gives, and the per-stream compaction follows."""
    tsb = rig["tsb"]
    parent = [-1, 0, 0, 1, 1, 2, 5]
    rng = np.random.default_rng(40 + streams)
    prompts = [rng.integers(0, rig["cfg"].vocab, size=9 + 2 * b).astype(np.int32) for b in range(streams)]  # ragged cursors
    feed = rng.integers(0, rig["cfg"].vocab, size=(streams, len(parent))).astype(np.int32)
    sess = tsb.Session(rig["ctx"], rig["target"], None, streams, 8)
    for b, pr in enumerate(prompts):
        for i, t in enumerate(pr):
            sess.produce_prefill(int(t), i, stream=b)
    single = []
    for b in range(streams):
        base = sess.checkpoint(stream=b)
        single.append(sess.verify_tree(feed[b], parent, base, stream=b).copy())
        sess.discard_pending(stream=b)
        assert sess.checkpoint(stream=b) == base
    batch = sess.verify_tree_streams(feed, parent)
    for b in range(streams):
        assert np.array_equal(batch[b], single[b]), b
    ost = oracle.State(rig["ot"])
    ost.forward(prompts[1], 0, want_logits=False)
    _close(oracle, batch[1], ost.forward(feed[1], len(prompts[1]), parent=parent), rel=4e-3, abs_=4e-3)
    # each stream finishes its round on its own: stream 1 keeps the path 0 -> 2 -> 5 -> 6
    base = len(prompts[1])
    sess.compact_tree(base, [0, 2, 5, 6], stream=1)
    sess.rollback_retaining(base, 4, stream=1)
    sess.commit_pending(4, stream=1)
    assert sess.checkpoint(stream=1) == base + 4
    ost.cursor = base
    ost.forward([int(feed[1][j]) for j in (0, 2, 5, 6)], base, want_logits=False)
    _close(oracle, sess.produce(11, base + 4, stream=1), ost.forward([11], base + 4)[0], rel=4e-3, abs_=4e-3)
    sess.close()


def test_rollback_retaining_after_a_tree_verify_needs_the_compaction_first(rig, oracle):
    tsb = rig["tsb"]
    sess = tsb.Session(rig["ctx"], rig["target"], rig["draft"], 1, 8)
    for i in range(10):
        sess.produce_prefill(3 + i, i)
    base = sess.checkpoint()
    sess.verify_tree([1, 2, 3, 4], [-1, 0, 0, 1], base)
    with pytest.raises(tsb.TsbError):
        sess.rollback_retaining(base, 2)  # the record of fed tokens ends at base: nothing says which slots to keep
    # discard_pending (crates/runtime/src/producer.rs:346-350) puts the stream back where the verify started
    sess.discard_pending()
    assert sess.checkpoint() == base
    a = sess.verify([1, 2, 3], base)
    sess.discard_pending()
    assert sess.checkpoint() == base
    b = sess.verify([1, 2, 3], base)
    assert np.array_equal(a, b)
    sess.commit_pending(3)
    sess.commit_pending(3)  # nothing pending: a no-op, as in the reference
    assert sess.supports_retaining_rollback() and sess.supports_headless_prefill() and not sess.drafts_block_passes()
    sess.close()


def _argmax(oracle, row16):
    v = oracle.f16_bits_to_f32(row16)
    return int(np.flatnonzero(v == v.max())[0])


@pytest.mark.parametrize("shape", [dict(nodes=10, branching=(2, 2, 1)), dict(nodes=9, levels=3, best_first=True, cand=3)])
def test_tree_rounds_driven_through_the_producer_calls_equal_the_sequential_loop(rig, oracle, shape):
    """The reference's round loop (crates/runtime/src/speculative.rs:461-575) written against the producer calls -
    tree_nodes, draft_tree, verify_tree, the accept walk, compact_tree, rollback_retaining, commit_pending,
    record_committed, rewind_drafter - must leave what greedy sequential decoding leaves, for the static shape and for
    the best-first tree."""
    tsb = rig["tsb"]
    sess = tsb.Session(rig["ctx"], rig["target"], rig["draft"], 1, 16)
    rng = np.random.default_rng(31)
    prompt = rng.integers(0, rig["cfg"].vocab, size=20).astype(np.int32)
    budget = 30
    _, want, _ = sess.sequential_run(prompt, tsb.run_config(tsb.shaping(temperature=0.0), budget, 3))
    sess.reset()
    assert sess.tree_nodes() is None
    with pytest.raises(tsb.TsbError):
        sess.draft_tree(1, 5, 4)  # chains only until a tree shape is set
    sess.set_tree(**shape)
    nodes = sess.tree_nodes()
    assert nodes == shape["nodes"]
    for i, t in enumerate(prompt[:-1]):
        sess.produce_prefill(int(t), i)
    logits = sess.produce(int(prompt[-1]), len(prompt) - 1)
    sess.prime_drafter(int(prompt[-1]), len(prompt) - 2)
    history = list(prompt)
    emitted = []
    nxt = _argmax(oracle, logits)
    accepted_total, first_round = 0, True
    while len(emitted) < budget:
        emitted.append(nxt)
        if len(emitted) == budget:
            break
        history.append(nxt)
        base = len(history) - 1
        if budget - len(emitted) < 3:  # not enough room for a full-depth tree: plain steps (the loop's truncated rounds)
            logits = sess.produce(nxt, base)
            sess.rewind_drafter(base)
            nxt = _argmax(oracle, logits)
            continue
        depth, cand, parent, toks = sess.draft_tree(nxt, base, nodes)
        assert all(p < i for i, p in enumerate(parent))  # parents precede children
        if first_round:
            # the first node is the drafter's most likely token after the anchor: what one greedy draft step proposes
            ref = tsb.Session(rig["ctx"], rig["target"], rig["draft"], 1, 16)
            for i, t in enumerate(history[:-1]):
                ref.produce_prefill(int(t), i)
            assert int(toks[0]) == _argmax(oracle, ref.draft_step(nxt, base - 1)) and depth[0] == 0 and parent[0] == -1
            ref.close()
            first_round = False
        slot_parent = np.array([-1] + [int(p) + 1 for p in parent], dtype=np.int32)  # dflash_tree_slot_parents
        feed = np.concatenate([[nxt], toks]).astype(np.int32)
        point = sess.checkpoint()
        rows = sess.verify_tree(feed, slot_parent, base)
        path, at, bonus = [0], -1, None
        while True:
            pick = _argmax(oracle, rows[at + 1])
            hit = [i for i in range(len(toks)) if parent[i] == at and toks[i] == pick]
            if not hit or len(emitted) + 1 >= budget:
                bonus = pick
                break
            path.append(hit[0] + 1)
            at = hit[0]
            emitted.append(pick)
            history.append(pick)
        committed = len(path) - 1
        accepted_total += committed
        sess.compact_tree(base, path)
        if committed + 1 < len(feed):
            sess.rollback_retaining(point, committed + 1)
        sess.commit_pending(committed + 1)
        sess.record_committed([int(feed[s]) for s in path], base)
        sess.rewind_drafter(base + committed)
        nxt = bonus
    assert emitted == list(want)
    sess.close()


def test_best_first_tree_rounds_in_the_library_loop_equal_the_sequential_loop(rig, oracle):
    tsb = rig["tsb"]
    sess = tsb.Session(rig["ctx"], rig["target"], rig["draft"], 1, 16)
    rng = np.random.default_rng(5)
    prompt = rng.integers(0, rig["cfg"].vocab, size=24).astype(np.int32)
    plain = tsb.run_config(tsb.shaping(temperature=0.0), 36, 3)
    tree = tsb.run_config(tsb.shaping(temperature=0.0), 36, 3, tree_nodes=8, tree_best_first=True, tree_cand=3, tree_levels=3)
    _, seq_emit, _ = sess.sequential_run(prompt, plain)
    _, emit, res = sess.spec_run(prompt, tree)
    assert np.array_equal(seq_emit, emit) and res.new_tokens == 36
    sess.close()


def test_draft_block_gives_the_greedy_chain_of_draft_steps(rig, oracle):
    tsb = rig["tsb"]
    sess = tsb.Session(rig["ctx"], rig["target"], rig["draft"], 1, 8)
    prompt = [4, 9, 200, 31, 77, 5]
    for i, t in enumerate(prompt):
        sess.produce_prefill(t, i)
    base = len(prompt) - 1  # the anchor's position; the drafter catches up to it from the record of fed tokens
    block = sess.draft_block(prompt[-1], base, 4)
    # the same through single steps on a second session
    ref = tsb.Session(rig["ctx"], rig["target"], rig["draft"], 1, 8)
    for i, t in enumerate(prompt):
        ref.produce_prefill(t, i)
    tok, want = prompt[-1], []
    for i in range(4):
        tok = _argmax(oracle, ref.draft_step(tok, base + i - 1))
        want.append(tok)
    assert list(block) == want
    sess.close(), ref.close()


@pytest.mark.parametrize("block", [1, 4])
def test_greedy_speculative_equals_greedy_sequential_token_for_token(rig, oracle, block):
    tsb = rig["tsb"]
    sess = tsb.Session(rig["ctx"], rig["target"], rig["draft"], 1, 16)
    rng = np.random.default_rng(1)
    prompt = rng.integers(0, rig["cfg"].vocab, size=32).astype(np.int32)
    rc = tsb.run_config(tsb.shaping(temperature=0.0), 48, block)
    seq_hist, seq_emit, seq_res = sess.sequential_run(prompt, rc)
    spec_hist, spec_emit, spec_res = sess.spec_run(prompt, rc)
    assert np.array_equal(seq_emit, spec_emit) and np.array_equal(seq_hist, spec_hist)
    assert spec_res.new_tokens == 48 and spec_res.reason == 0 and spec_res.kv_position == spec_res.history_len
    assert spec_res.rounds <= 48
    # and against the CPU oracle's own loop over its own forward pass
    orc = oracle.run_config(oracle.shaping(temperature=0.0), 48, block)
    oh, oe, ores = oracle.run_speculative_model(oracle.State(rig["ot"]), oracle.State(rig["od"]), prompt, orc)
    # token-identical up to the first near-tie: where the two streams part, the oracle's own logits must show
    # the two candidates within the matmul tolerance of each other (a different summation order flipped an argmax)
    n_same = 0
    while n_same < len(oe) and oe[n_same] == spec_emit[n_same]:
        n_same += 1
    assert n_same >= 8, n_same
    if n_same < len(oe):
        ost = oracle.State(rig["ot"])
        ctx_tokens = list(prompt) + [int(t) for t in oe[:n_same]]
        lg = oracle.f16_bits_to_f32(ost.forward(ctx_tokens, 0)[-1])
        gap = lg[int(oe[n_same])] - lg[int(spec_emit[n_same])]
        assert 0 <= gap <= 2 * (4e-3 + 4e-3 * abs(lg[int(oe[n_same])])), (n_same, gap)
    sess.close()


def test_the_timing_aids_leave_the_committed_state_alone(rig, oracle):
    """tsb_session_time_matmuls and tsb_session_time_pass_rest enqueue a pass's launches over rows past the cursor:
    afterwards the next logits are the bits they would have been without the calls."""
    tsb = rig["tsb"]
    rng = np.random.default_rng(5)
    prompt = rng.integers(0, rig["cfg"].vocab, size=20).astype(np.int32)
    sess = tsb.Session(rig["ctx"], rig["target"], rig["draft"], 1, 8)
    for i, t in enumerate(prompt[:-1]):
        sess.produce(int(t), i)
    want = None
    for timed in (False, True):
        if timed:
            ms, nbytes, launches = sess.time_matmuls(6, 2)
            rest = sess.time_pass_rest(6, 2)
            assert ms > 0 and rest > 0 and nbytes > 0 and launches >= 4 * rig["cfg"].n_layers
        point = sess.checkpoint()
        got = sess.produce(int(prompt[-1]), point)
        sess.rollback_retaining(point, 0)
        if want is None:
            want = got
        else:
            assert np.array_equal(got, want)
    sess.close()


def test_sampled_round_decisions_match_the_oracle_given_the_devices_logits(rig, oracle):
    tsb = rig["tsb"]
    ctx = rig["ctx"]
    K = 4
    sess = tsb.Session(ctx, rig["target"], rig["draft"], 1, K + 1)
    rng = np.random.default_rng(3)
    prompt = rng.integers(0, rig["cfg"].vocab, size=16).astype(np.int32)
    for i, t in enumerate(prompt[:-1]):
        sess.produce_prefill(int(t), i)
    sess.produce(int(prompt[-1]), len(prompt) - 1)
    sess.prime_drafter(int(prompt[-1]), len(prompt) - 2)
    rc = tsb.run_config(tsb.shaping(temperature=1.0, seed=2), 64, K, uniform_mode=1)
    nxt = np.array([123], dtype=np.int32)
    steps = np.zeros(1, dtype=np.uint64)
    ocfg = oracle.shaping(temperature=1.0, seed=2)
    for rnd in range(6):
        base = sess.checkpoint()
        step0 = int(steps[0])
        confirmed = int(nxt[0])
        accepted = sess.round(rc, nxt, steps)[0]
        # replay the round through the single-stream producer calls to obtain the logits the kernels saw
        sess.kv(0).set_cursor(0, base)
        sess.kv(1).set_cursor(0, base)
        chained, props, dlogits = confirmed, [], []
        for d in range(K):
            lg = sess.draft_step(chained, base - 1 + d)
            tok, _ = oracle.sample(lg, ocfg, oracle.uniform_u64(1, 2, step0 + d))
            dlogits.append(lg), props.append(tok)
            chained = tok
        tlogits = sess.verify([confirmed] + props, base)
        unis = [oracle.uniform_u64(1, 2, step0 + K + 1 + j) for j in range(2 * K + 1)]
        acc, toks, draws, margins = oracle.accept_round(tlogits, np.stack(dlogits), props, ocfg, unis)
        assert acc == accepted and toks[-1] == nxt[0], (rnd, acc, accepted, toks, nxt)
        assert int(steps[0]) == step0 + K + 1 + draws
        sess.kv(0).set_cursor(0, base + acc + 1)
        sess.kv(1).set_cursor(0, base + acc + 1)
    sess.close()


def test_penalised_rounds_match_the_oracle_given_the_devices_logits(rig, oracle):
    """Repetition, presence and frequency penalties inside the round: every proposal is shaped with the history the
    round started with, target row i with the history grown by the proposals accepted before it
    (crates/runtime/src/speculative.rs:636-648,701-734); decisions, tokens and draw counts equal the oracle's on the
    logits the kernels saw, and they differ from the unpenalised ones (the test is not vacuous)."""
    tsb = rig["tsb"]
    ctx = rig["ctx"]
    K = 4
    sess = tsb.Session(ctx, rig["target"], rig["draft"], 1, K + 1)
    rng = np.random.default_rng(13)
    prompt = rng.integers(0, rig["cfg"].vocab, size=24).astype(np.int32)
    for i, t in enumerate(prompt[:-1]):
        sess.produce_prefill(int(t), i)
    sess.produce(int(prompt[-1]), len(prompt) - 1)
    sess.prime_drafter(int(prompt[-1]), len(prompt) - 2)
    pen = dict(temperature=1.0, seed=2, repetition_penalty=1.4, presence_penalty=0.6, frequency_penalty=0.3)
    rc = tsb.run_config(tsb.shaping(**pen), 64, K, uniform_mode=1)
    ocfg, plain = oracle.shaping(**pen), oracle.shaping(temperature=1.0, seed=2)
    nxt = np.array([int(prompt[3])], dtype=np.int32)  # a token that is already in the history
    steps = np.zeros(1, dtype=np.uint64)
    history, gen = list(map(int, prompt)), 1
    sess.set_generated(gen)
    moved = 0
    for rnd in range(6):
        base = sess.checkpoint()
        step0 = int(steps[0])
        confirmed = int(nxt[0])
        hist0 = history + [confirmed]
        accepted = sess.round(rc, nxt, steps)[0]
        sess.kv(0).set_cursor(0, base)
        sess.kv(1).set_cursor(0, base)
        chained, props, dlogits = confirmed, [], []
        for d in range(K):
            lg = sess.draft_step(chained, base - 1 + d)
            tok, _ = oracle.sample(lg, ocfg, oracle.uniform_u64(1, 2, step0 + d), history=hist0, generated=gen)
            moved += tok != oracle.sample(lg, plain, oracle.uniform_u64(1, 2, step0 + d))[0]
            dlogits.append(lg), props.append(tok)
            chained = tok
        tlogits = sess.verify([confirmed] + props, base)
        unis = [oracle.uniform_u64(1, 2, step0 + K + 1 + j) for j in range(2 * K + 1)]
        acc, toks, draws, _ = oracle.accept_round(tlogits, np.stack(dlogits), props, ocfg, unis, history=hist0, generated=gen)
        assert acc == accepted and toks[-1] == nxt[0], (rnd, acc, accepted, toks, nxt)
        assert int(steps[0]) == step0 + K + 1 + draws
        sess.kv(0).set_cursor(0, base + acc + 1)
        sess.kv(1).set_cursor(0, base + acc + 1)
        history = hist0 + [int(t) for t in toks[:acc]]
        gen += acc + 1
    assert moved > 0
    sess.close()


def test_penalised_generation_loops_run_and_agree_on_the_first_token(rig, oracle):
    """The loops take a shaping record with penalties (they refused it before): the sequential loop's tokens equal the
    oracle's select over the device logits with the growing history, and the speculative loop starts from the same token."""
    tsb = rig["tsb"]
    sess = tsb.Session(rig["ctx"], rig["target"], rig["draft"], 1, 8)
    rng = np.random.default_rng(17)
    prompt = rng.integers(0, rig["cfg"].vocab, size=12).astype(np.int32)
    pen = dict(temperature=0.9, seed=5, repetition_penalty=1.3, presence_penalty=0.5, frequency_penalty=0.25, top_k=40)
    rc = tsb.run_config(tsb.shaping(**pen), 10, 3)
    hist, emitted, res = sess.sequential_run(prompt, rc)
    assert res.new_tokens == 10
    # replay: feed the same tokens and select with the oracle on the device's logits
    ocfg = oracle.shaping(**pen)
    sess.reset()
    for i, t in enumerate(prompt[:-1]):
        sess.produce_prefill(int(t), i)
    logits = sess.produce(int(prompt[-1]), len(prompt) - 1)
    history = list(map(int, prompt))
    for g in range(10):
        tok, _ = oracle.sample(logits, ocfg, oracle.uniform_u64(0, 5, g), history=history, generated=g)
        assert tok == int(emitted[g]), (g, tok, int(emitted[g]))
        history.append(tok)
        if g < 9:
            logits = sess.produce(tok, len(history) - 1)
    _, spec_emitted, res2 = sess.spec_run(prompt, rc)
    assert res2.new_tokens == 10 and int(spec_emitted[0]) == int(emitted[0])
    sess.close()


def test_stop_token_budget_and_refusals(rig, oracle):
    tsb = rig["tsb"]
    sess = tsb.Session(rig["ctx"], rig["target"], rig["draft"], 1, 8)
    rng = np.random.default_rng(5)
    prompt = rng.integers(0, rig["cfg"].vocab, size=8).astype(np.int32)
    rc = tsb.run_config(tsb.shaping(temperature=0.0), 24, 3)
    _, emitted, _ = sess.sequential_run(prompt, rc)
    stop_tok = int(emitted[9])
    rc2 = tsb.run_config(tsb.shaping(temperature=0.0), 24, 3, stop_tokens=(stop_tok,))
    h1, e1, r1 = sess.sequential_run(prompt, rc2)
    h2, e2, r2 = sess.spec_run(prompt, rc2)
    assert r1.reason == r2.reason == 1 and np.array_equal(e1, e2) and np.array_equal(h1, h2)
    assert e2[-1] == stop_tok and len(h2) == len(prompt) + len(e2) - 1  # the stopping token is counted, not fed
    for bad in (tsb.run_config(tsb.shaping(temperature=0.0), 24, 0), tsb.run_config(tsb.shaping(temperature=0.0), 0, 2),
                tsb.run_config(tsb.shaping(temperature=0.0), 600, 2), tsb.run_config(tsb.shaping(temperature=0.7, repetition_penalty=0.0), 8, 2)):
        with pytest.raises(tsb.TsbError):
            sess.spec_run(prompt, bad)
    with pytest.raises(tsb.TsbError):
        sess.spec_run(np.zeros(0, np.int32), rc)
    sess.close()


@pytest.mark.parametrize("nodes,branching", [(10, (2, 2, 1)), (14, (2, 2, 2)), (6, (3, 1))])
def test_greedy_tree_rounds_equal_the_sequential_loop_token_for_token(rig, oracle, nodes, branching):
    """Static-tree rounds: drafter top-b children per level, one tree verify, the accept walk and in-place compaction
    must leave exactly what greedy sequential decoding leaves (crates/runtime/src/speculative.rs:461-560)."""
    tsb = rig["tsb"]
    sess = tsb.Session(rig["ctx"], rig["target"], rig["draft"], 1, 16)
    rng = np.random.default_rng(21)
    prompt = rng.integers(0, rig["cfg"].vocab, size=24).astype(np.int32)
    plain = tsb.run_config(tsb.shaping(temperature=0.0), 40, len(branching))
    tree = tsb.run_config(tsb.shaping(temperature=0.0), 40, len(branching), tree_nodes=nodes, tree_branching=branching)
    seq_hist, seq_emit, _ = sess.sequential_run(prompt, plain)
    hist, emit, res = sess.spec_run(prompt, tree)
    assert np.array_equal(seq_emit, emit) and np.array_equal(seq_hist, hist)
    assert res.new_tokens == 40 and res.kv_position == res.history_len
    # a tree offers the chain's first proposal among others, so it accepts at least as much as the chain does
    _, _, chain = sess.spec_run(prompt, plain)
    assert res.accepted_total >= chain.accepted_total and res.rounds <= chain.rounds
    # refusals: sampled tree rounds, block != levels, a tree larger than the session's rows
    for bad in (tsb.run_config(tsb.shaping(temperature=1.0), 8, len(branching), tree_nodes=nodes, tree_branching=branching),
                tsb.run_config(tsb.shaping(temperature=0.0), 8, len(branching) + 1, tree_nodes=nodes, tree_branching=branching),
                tsb.run_config(tsb.shaping(temperature=0.0), 8, 2, tree_nodes=40, tree_branching=(8, 8))):
        with pytest.raises(tsb.TsbError):
            sess.spec_run(prompt, bad)
    sess.close()


def test_prefix_reuse_keeps_the_shared_rows_and_changes_nothing_else(rig, oracle):
    """try_reuse_prefix (crates/runtime/src/producer.rs:21-47): a second prompt that repeats the first turn's history
    and adds to it keeps the cache rows of the common prefix; the output equals a run from an empty cache."""
    tsb = rig["tsb"]
    sess = tsb.Session(rig["ctx"], rig["target"], rig["draft"], 1, 16)
    rng = np.random.default_rng(9)
    prompt = rng.integers(0, rig["cfg"].vocab, size=40).astype(np.int32)
    rc = tsb.run_config(tsb.shaping(temperature=0.0), 24, 3)
    h1, _, r1 = sess.spec_run(prompt, rc)
    assert r1.reused_prefix == 0
    # second turn: the first turn's history (as committed) plus new tokens
    turn2 = np.concatenate([h1, rng.integers(0, rig["cfg"].vocab, size=12).astype(np.int32)])
    reuse = tsb.run_config(tsb.shaping(temperature=0.0), 24, 3, reuse_prefix=True)
    h2, e2, r2 = sess.spec_run(turn2, reuse)
    assert r2.reused_prefix == len(h1)  # every committed row of the first turn was kept
    fresh = tsb.Session(rig["ctx"], rig["target"], rig["draft"], 1, 16)
    h3, e3, r3 = fresh.spec_run(turn2, rc)
    assert np.array_equal(e2, e3) and np.array_equal(h2, h3)
    # a prompt that diverges inside the cached part keeps only the common prefix
    turn3 = turn2.copy()
    turn3[10] = (turn3[10] + 1) % rig["cfg"].vocab
    _, e4, r4 = sess.spec_run(turn3, reuse)
    assert r4.reused_prefix == 10
    _, e5, _ = fresh.spec_run(turn3, rc)
    assert np.array_equal(e4, e5)
    # the sequential loop takes the same option
    _, e6, r6 = sess.sequential_run(turn3, reuse)
    assert r6.reused_prefix > 0 and np.array_equal(e6, e5)
    sess.close(), fresh.close()


def test_many_row_passes_match_the_oracle_forward(rig, oracle):
    """Passes of 24 rows and more run the matmuls on tensor memory with the reference's own operator order; a 40-row
    chain verify and a 33-row tree verify must match the oracle's forward within the matmul tolerance."""
    tsb = rig["tsb"]
    sess = tsb.Session(rig["ctx"], rig["target"], rig["draft"], 1, 48)
    ost = oracle.State(rig["ot"])
    rng = np.random.default_rng(17)
    prompt = rng.integers(0, rig["cfg"].vocab, size=30).astype(np.int32)
    for i, t in enumerate(prompt):
        sess.produce_prefill(int(t), i)
    ost.forward(prompt, 0, want_logits=False)
    feed = rng.integers(0, rig["cfg"].vocab, size=40).astype(np.int32)
    base = sess.checkpoint()
    got = sess.verify(feed, base)
    want = ost.forward(feed, base)
    _close(oracle, got, want, rel=4e-3, abs_=4e-3)
    # the same rows a few at a time (register-MMA path) agree with the many-row pass within the same tolerance
    sess.rollback_retaining(base, 0)
    few = np.concatenate([sess.verify(feed[i:i + 8], base + i) for i in range(0, 40, 8)])
    _close(oracle, got, few, rel=4e-3, abs_=4e-3)
    # a tree of 32 nodes + anchor
    sess.rollback_retaining(base, 0)
    ost.cursor = base
    parent = [-1] + [max(0, (i - 1) // 2) for i in range(1, 33)]
    tfeed = rng.integers(0, rig["cfg"].vocab, size=33).astype(np.int32)
    got_t = sess.verify_tree(tfeed, parent, base)
    want_t = ost.forward(tfeed, base, parent=parent)
    _close(oracle, got_t, want_t, rel=4e-3, abs_=4e-3)
    sess.close()


@pytest.mark.parametrize("S,K", [(3, 3), (4, 5), (6, 5)])
def test_lockstep_rounds_over_several_streams_equal_single_stream_runs(rig, oracle, S, K):
    """Independent streams in one session: every stream's greedy output from lockstep rounds equals its own sequential
    run (streams of different lengths, different prompts).  With 4 streams at K = 5 the verify pass carries 24 rows and
    the session's target runs the tensor-memory matmul - for every pass, the single-row decodes of the sequential loop
    included, so the two loops still agree token for token."""
    tsb = rig["tsb"]
    NEW = 20
    sess = tsb.Session(rig["ctx"], rig["target"], rig["draft"], S, K + 1)
    solo = sess  # the sequential runs use the same session: one matmul path per (session, model)
    rng = np.random.default_rng(33)
    prompts = [rng.integers(0, rig["cfg"].vocab, size=n).astype(np.int32) for n in (9, 21, 14, 30, 12, 17)[:S]]
    rc = tsb.run_config(tsb.shaping(temperature=0.0), 1 << 20, K)
    want = [solo.sequential_run(p, tsb.run_config(tsb.shaping(temperature=0.0), NEW, K), stream=q)[1] for q, p in enumerate(prompts)]
    nxt = np.zeros(S, dtype=np.int32)
    for q, p in enumerate(prompts):
        sess.reset(stream=q)
        for i, t in enumerate(p[:-1]):
            sess.produce_prefill(int(t), i, stream=q)
        lg = oracle.f16_bits_to_f32(sess.produce(int(p[-1]), len(p) - 1, stream=q))
        nxt[q] = int(np.argmax(lg))
        sess.prime_drafter(int(p[-1]), len(p) - 2, stream=q)
    out = [[] for _ in range(S)]
    steps = np.zeros(S, dtype=np.uint64)
    for _ in range(NEW):
        confirmed = nxt.copy()
        acc, toks = sess.round_tokens(rc, nxt, steps)
        for q in range(S):
            out[q].append(int(confirmed[q]))
            out[q].extend(int(t) for t in toks[q, :acc[q]])
            assert toks[q, acc[q]] == nxt[q]
    for q in range(S):
        assert out[q][:NEW] == list(want[q][:NEW]), (q, out[q][:NEW], list(want[q][:NEW]))
    sess.close()


def test_penalised_lockstep_rounds_over_streams_equal_each_streams_own_rounds(rig, oracle):
    """Three streams with different histories in one penalised round sequence: every stream's accepted counts and
    tokens equal those of the same stream driven alone (its history row on the device is its own, whatever its place
    in the batch)."""
    tsb = rig["tsb"]
    S, K, ROUNDS = 3, 3, 5
    pen = dict(temperature=1.0, seed=9, repetition_penalty=1.5, presence_penalty=0.7, frequency_penalty=0.2)
    rc = tsb.run_config(tsb.shaping(**pen), 1 << 20, K, uniform_mode=1)
    rng = np.random.default_rng(55)
    prompts = [rng.integers(0, rig["cfg"].vocab, size=n).astype(np.int32) for n in (10, 17, 13)]

    def start(sess, q, p):
        sess.reset(stream=q)
        for i, t in enumerate(p[:-1]):
            sess.produce_prefill(int(t), i, stream=q)
        sess.produce(int(p[-1]), len(p) - 1, stream=q, want_logits=False)
        sess.prime_drafter(int(p[-1]), len(p) - 2, stream=q)
        sess.set_generated(1, stream=q)

    sess = tsb.Session(rig["ctx"], rig["target"], rig["draft"], S, K + 1)
    for q, p in enumerate(prompts):
        start(sess, q, p)
    nxt = np.array([int(p[2]) for p in prompts], dtype=np.int32)
    steps = np.zeros(S, dtype=np.uint64)
    together = []
    for _ in range(ROUNDS):
        acc, toks = sess.round_tokens(rc, nxt, steps)
        together.append((acc.copy(), toks.copy(), nxt.copy()))
    sess.close()
    # a stream's seed is the record's seed plus its index: alone in a one-stream session it sits at index 0
    for q, p in enumerate(prompts):
        solo = tsb.Session(rig["ctx"], rig["target"], rig["draft"], 1, K + 1)
        start(solo, 0, p)
        rcq = tsb.run_config(tsb.shaping(**dict(pen, seed=pen["seed"] + q)), 1 << 20, K, uniform_mode=1)
        n1 = np.array([int(p[2])], dtype=np.int32)
        s1 = np.zeros(1, dtype=np.uint64)
        for r in range(ROUNDS):
            acc, toks = solo.round_tokens(rcq, n1, s1)
            assert acc[0] == together[r][0][q] and np.array_equal(toks[0], together[r][1][q]) and n1[0] == together[r][2][q], (q, r)
        solo.close()


def test_prefix_reuse_with_a_long_prompt_equals_a_cold_run_on_the_many_row_path(rig, oracle):
    """A session whose largest pass has 24 rows or more prefills in chunks of that size; a later turn that reuses a
    prefix prefills in other chunk sizes.  One matmul path per (session, model) keeps the cache rows - and the
    output - identical to a run from an empty cache."""
    tsb = rig["tsb"]
    sess = tsb.Session(rig["ctx"], rig["target"], rig["draft"], 1, 32)
    rng = np.random.default_rng(41)
    prompt = rng.integers(0, rig["cfg"].vocab, size=70).astype(np.int32)
    rc = tsb.run_config(tsb.shaping(temperature=0.0), 16, 3)
    h1, _, _ = sess.spec_run(prompt, rc)
    turn2 = np.concatenate([h1, rng.integers(0, rig["cfg"].vocab, size=29).astype(np.int32)])
    _, e2, r2 = sess.spec_run(turn2, tsb.run_config(tsb.shaping(temperature=0.0), 16, 3, reuse_prefix=True))
    assert r2.reused_prefix == len(h1)
    cold = tsb.Session(rig["ctx"], rig["target"], rig["draft"], 1, 32)
    _, e3, _ = cold.spec_run(turn2, rc)
    assert np.array_equal(e2, e3)
    sess.close(), cold.close()


def test_adaptive_depth_changes_the_round_shape_not_the_output(rig, oracle):
    """AdaptiveDepth (crates/runtime/src/speculative_adaptive.rs:104-225) only picks how many proposals a round offers:
    greedy output stays token-identical to the sequential loop, and a run that starts at the floor offers less per
    round than a fixed-depth run."""
    tsb = rig["tsb"]
    sess = tsb.Session(rig["ctx"], rig["target"], rig["draft"], 1, 16)
    rng = np.random.default_rng(44)
    prompt = rng.integers(0, rig["cfg"].vocab, size=20).astype(np.int32)
    fixed = tsb.run_config(tsb.shaping(temperature=0.0), 48, 5)
    adaptive = tsb.run_config(tsb.shaping(temperature=0.0), 48, 5, adaptive=2)
    _, seq, _ = sess.sequential_run(prompt, fixed)
    _, e_fixed, r_fixed = sess.spec_run(prompt, fixed)
    _, e_adapt, r_adapt = sess.spec_run(prompt, adaptive)
    assert np.array_equal(seq, e_fixed) and np.array_equal(seq, e_adapt)
    assert r_adapt.new_tokens == 48 and r_adapt.rounds >= r_fixed.rounds
    sess.close()


@pytest.mark.parametrize("order,recipe_name", [(None, "q4_k_m"), ("v_first", "q4_k_m"), (None, "q5_k_m")])
def test_mixed_recipe_layers_match_the_oracle(oracle, order, recipe_name):
    """Mixed recipes.  q4_k_m: q, k, o, gate, up in Q4_K; v, down and the head in Q6_K.  q5_k_m: Q5_K in place of
    Q4_K and a Q8_0 embedding table.  v sits in its own matrix and runs as a second launch; the logits must match
    the oracle's forward pass over the same blocks, whichever of q, k, v is uploaded first."""
    import turbospark_b200 as tsb
    from turbospark_b200.model import W_Q, W_V, W_DOWN, W_EMBED, W_LM_HEAD
    ctx = tsb.Ctx(0)
    cfg = tsb.config_tiny(max_context=256)
    recipe = {W_V: tsb.Q6_K, W_DOWN: tsb.Q6_K, W_LM_HEAD: tsb.Q6_K}
    base = tsb.Q4_K
    if recipe_name == "q5_k_m":
        recipe[W_EMBED] = tsb.Q8_0
        base = tsb.Q5_K
    mats, norms = weights.random_weights(cfg, 5, oracle, qtype=base, real_ffn=1408, qtype_of=recipe)
    target = tsb.Model(ctx, cfg)
    weights.load_weights(target, mats, norms, order=[W_V] if order else None)
    assert target.weight_bytes == sum(b.size for (l, w), (b, _, _, _) in mats.items() if w != W_EMBED)
    ocfg = oracle.ModelCfg(cfg.n_layers, cfg.d_model, cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim, cfg.ffn, cfg.vocab,
                           cfg.max_context, cfg.rms_eps, cfg.rope_theta)
    ot = oracle.Model(ocfg, threads=8)
    weights.load_weights(ot, mats, norms)
    sess = tsb.Session(ctx, target, None, 1, 8)
    ost = oracle.State(ot)
    rng = np.random.default_rng(9)
    prompt = rng.integers(0, cfg.vocab, size=10).astype(np.int32)
    for i, t in enumerate(prompt):
        _close(oracle, sess.produce(int(t), i), ost.forward([int(t)], i)[0], rel=4e-3, abs_=4e-3)
    feed = rng.integers(0, cfg.vocab, size=6).astype(np.int32)
    point = sess.checkpoint()
    _close(oracle, sess.verify(feed, point), ost.forward(feed, point), rel=4e-3, abs_=4e-3)
    # q in a format other than k is still refused
    with pytest.raises(tsb.TsbError):
        qb = oracle.quantize(tsb.Q6_K, np.zeros((cfg.n_q_heads * cfg.head_dim, cfg.d_model), np.float32))
        target.set_matrix(0, W_Q, tsb.Q6_K, qb, cfg.n_q_heads * cfg.head_dim, cfg.d_model)
    sess.close(), target.close(), ctx.close()


def test_a_model_loaded_from_a_resident_weight_file_gives_the_same_logits(oracle, tmp_path):
    """The install-side path: a mixed-recipe tensor set written in the resident file layout under the names the
    reference's Llama runner looks up, read back through the index and uploaded verbatim."""
    import turbospark_b200 as tsb
    from turbospark_b200 import resident
    from turbospark_b200.model import W_V, W_DOWN, W_LM_HEAD, W_Q
    ctx = tsb.Ctx(0)
    cfg = tsb.config_tiny(max_context=256)
    mats, norms = weights.random_weights(cfg, 6, oracle, real_ffn=1408, qtype_of={W_V: tsb.Q6_K, W_DOWN: tsb.Q6_K, W_LM_HEAD: tsb.Q6_K})
    direct = tsb.Model(ctx, cfg)
    weights.load_weights(direct, mats, norms)
    path = tmp_path / "model_weights.bin"
    path.write_bytes(resident.build_resident_file(resident.llama_tensor_list(cfg, mats, norms)))
    idx = resident.ResidentIndex(path)
    assert len(idx) == 2 + cfg.n_layers * 9 + 1
    loaded = tsb.Model(ctx, cfg)
    idx.load_into(loaded)
    assert loaded.weight_bytes == direct.weight_bytes
    rng = np.random.default_rng(3)
    feed = rng.integers(0, cfg.vocab, size=6).astype(np.int32)
    outs = []
    for m in (direct, loaded):
        sess = tsb.Session(ctx, m, None, 1, 8)
        outs.append(sess.verify(feed, 0).copy())
        sess.close()
    assert np.array_equal(outs[0], outs[1])
    # a tensor whose byte count does not fit the model's shape is refused, as is a non-block dtype
    wrong = tsb.Model(ctx, tsb.ModelConfig(cfg.n_layers, cfg.d_model, cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim, cfg.ffn,
                                           cfg.vocab * 2, cfg.max_context, cfg.rms_eps, cfg.rope_theta))
    with pytest.raises(tsb.TsbError, match="does not match"):
        idx.load_into(wrong)
    tensors = resident.llama_tensor_list(cfg, mats, norms)
    tensors[2] = (tensors[2][0], 1, tensors[2][2], tensors[2][3])      # layer 0 q_proj tagged BF16
    bad = tmp_path / "bad.bin"
    bad.write_bytes(resident.build_resident_file(tensors))
    with pytest.raises(tsb.TsbError, match="dtype tag"):
        resident.ResidentIndex(bad).load_into(tsb.Model(ctx, cfg))
    idx.close(), direct.close(), loaded.close(), wrong.close(), ctx.close()
