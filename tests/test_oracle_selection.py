"""The CPU oracle's sampler and round loop against the reference's own worked examples.

Each case restates a test the reference holds (path within the reference project in the
comment), with the same input numbers, so the oracle is pinned before any kernel is
compared with it.
"""
import numpy as np
import pytest


def f16(oracle, values):
    return oracle.f32_to_f16_bits(np.asarray(values, dtype=np.float32))


def structured_scores(oracle):
    # crates/selection/tests/rejection_sampling.rs:14-28
    base = [-1.0 - i * 0.01 for i in range(64)]
    base[7], base[19], base[20], base[33] = 6.0, 4.5, 4.2, 3.0
    return f16(oracle, np.array(base, dtype=np.float32))


def test_derive_step_value_contract(oracle):
    # crates/selection/src/derive.rs:50-70
    assert oracle.derive_step_value(7, 3) == oracle.derive_step_value(7, 3)
    assert oracle.derive_step_value(7, 3) != oracle.derive_step_value(7, 4)
    for pos in range(50):
        v = oracle.to_unit_interval(oracle.derive_step_value(1, pos))
        assert 0.0 <= v < 1.0
    # the mixer is the splitmix64 finalizer: known value for x = 0
    # mix(0 ^ 0) = splitmix64 output for state 0
    assert oracle.derive_step_value(0, 0) == 0xE220A8397B1DCDAF


def test_residual_worked_examples(oracle):
    # crates/selection/src/distribution.rs:147-262
    r = oracle.residual(([0, 1], [0.5, 0.5]), ([0], [1.0]))
    assert list(r[0]) == [1] and r[1][0] == 1.0
    r = oracle.residual(([0, 1], [0.6, 0.4]), ([0, 1, 2], [0.2, 0.1, 0.7]))
    assert list(r[0]) == [0, 1]
    assert abs(r[1][0] - 0.4 / 0.7) < 1e-12 and abs(r[1][1] - 0.3 / 0.7) < 1e-12
    assert oracle.residual(([0, 1], [0.5, 0.5]), ([0, 1], [0.5, 0.5])) is None
    r = oracle.residual(([5], [1.0]), ([9], [1.0]))
    assert list(r[0]) == [5] and r[1][0] == 1.0
    # order and first-occurrence, bit for bit
    ps, pp = [9, 2, 40, 7, 1000], [0.3, 0.25, 0.2, 0.15, 0.1]
    qs, qp = [7, 40, 40, 2, 11], [0.05, 0.1, 0.6, 0.3, 0.05]
    first = {}
    for t, w in zip(qs, qp):
        first.setdefault(t, w)
    mass = [max(w - first.get(t, 0.0), 0.0) for t, w in zip(ps, pp)]
    total = 0.0
    for m in mass:
        if m > 0:
            total += m
    want = [(t, m / total) for t, m in zip(ps, mass) if m > 0]
    assert [t for t, _ in want] == [9, 40, 7, 1000]
    r = oracle.residual((ps, pp), (qs, qp))
    assert list(r[0]) == [t for t, _ in want]
    assert [float(x).hex() for x in r[1]] == [float(m).hex() for _, m in want]


def test_residual_at_full_vocabulary_keeps_p_order(oracle):
    n = 262144
    wsum = n * (n + 1.0) / 2.0
    sup = np.arange(n, dtype=np.uint32)
    probs = (np.arange(n, dtype=np.float64) + 1.0) / wsum
    r = oracle.residual((sup, probs), (sup[::-1].copy(), np.full(n, 1.0 / n)))
    assert np.array_equal(r[0], np.arange(n // 2, n, dtype=np.uint32))


def test_shaped_distribution_draws_what_select_draws(oracle):
    # crates/selection/tests/rejection_sampling.rs:42-74
    scores = structured_scores(oracle)
    history = [3, 7, 11]
    for (t, k, p, seed) in [(0.2, 64, 0.95, 7), (0.7, 0, 0.0, 9), (1.3, 8, 0.9, 11), (0.5, 64, 0.95, 20260911)]:
        cfg = oracle.shaping(temperature=t, top_k=k, top_p=p, seed=seed)
        for position in (0, 1, 2, 5, 17, 100):
            selected = oracle.select(scores, cfg, history, position)
            dist = oracle.shaped_distribution(scores, cfg, history, position)
            target = oracle.to_unit_interval(oracle.derive_step_value(seed, position))
            assert selected == oracle.draw(dist, target)


def test_distribution_is_normalized_and_covers_select(oracle):
    # crates/selection/tests/rejection_sampling.rs:76-104
    scores = structured_scores(oracle)
    cfg = oracle.shaping(temperature=0.8, top_k=16, top_p=0.95, seed=4242)
    sup, pr = oracle.shaped_distribution(scores, cfg, [3, 7, 11], 0)
    assert abs(pr.sum() - 1.0) < 1e-9
    for position in range(256):
        assert oracle.select(scores, cfg, [3, 7, 11], position) in set(int(s) for s in sup)


def test_deterministic_is_first_argmax_and_ignores_shaping(oracle):
    scores = f16(oracle, [1.0, 5.0, 5.0, -2.0])
    cfg = oracle.shaping(temperature=0.0, top_k=1, top_p=0.1, repetition_penalty=4.0, seed=5)
    assert oracle.select(scores, cfg, [1], 3) == 1
    sup, pr = oracle.shaped_distribution(scores, cfg, [1], 3)
    assert list(sup) == [1] and list(pr) == [1.0]


def test_rank_order_is_descending_with_ties_to_the_lower_index(oracle):
    # crates/selection/src/truncation.rs:79-99
    scores = f16(oracle, [0.5, 2.0, 2.0, -1.0, 2.0, 0.5])
    sup, pr = oracle.shaped_distribution(scores, oracle.shaping(temperature=1.0, seed=1))
    assert list(sup) == [1, 2, 4, 0, 5, 3]
    assert abs(pr.sum() - 1.0) < 1e-12
    # top-k keeps the prefix of the same order
    sup, _ = oracle.shaped_distribution(scores, oracle.shaping(temperature=1.0, top_k=2, seed=1))
    assert list(sup) == [1, 2]


def test_underflowed_exps_tie_by_index_not_by_logit(oracle):
    # logits far below the max underflow to exp == 0 and then order by index
    scores = f16(oracle, [-60000.0, 60000.0, -50000.0, -60000.0])
    sup, pr = oracle.shaped_distribution(scores, oracle.shaping(temperature=1.0, seed=1))
    assert list(sup) == [1, 0, 2, 3]
    assert pr[0] == 1.0


def test_penalties(oracle):
    # crates/selection/src/penalty.rs:84-177
    scores = f16(oracle, [4.0, -4.0, 1.0])
    cfg = oracle.shaping(temperature=1.0, repetition_penalty=2.0, seed=1)
    sup, pr = oracle.shaped_distribution(scores, cfg, [0, 1, 0], 0)
    # 4 -> 2, -4 -> -8, 1 stays: order 0, 2, 1
    assert list(sup) == [0, 2, 1]
    e = np.exp(np.array([0.0, -1.0, -10.0]))
    assert np.allclose(pr, e / e.sum(), rtol=1e-12)
    non_finite = f16(oracle, [1.0, np.inf])
    with pytest.raises(ValueError):
        oracle.select(non_finite, cfg)


def test_min_p_and_top_p_compose(oracle):
    scores = f16(oracle, [5.0, 4.0, 1.0, 0.0])
    sup, _ = oracle.shaped_distribution(scores, oracle.shaping(temperature=1.0, min_p=0.2, seed=1))
    assert list(sup) == [0, 1]
    sup, _ = oracle.shaped_distribution(scores, oracle.shaping(temperature=1.0, top_p=0.5, seed=1))
    assert list(sup) == [0]


def _scripted(oracle, quality, graded, speculative, temperature=0.0, block=4, max_new=64, seed=1, prompt_len=5,
              max_context=4096, stop=(), adaptive=0, vocab=97):
    cfg = oracle.shaping(temperature=temperature, top_k=64 if graded else 0, top_p=0.95 if graded else 0.0, seed=seed)
    rc = oracle.run_config(cfg, max_new, block, stop_tokens=stop, adaptive=adaptive)
    prompt = [(i * 5 + 1) % vocab for i in range(prompt_len)]
    return oracle.run_scripted(vocab, quality, graded, speculative, prompt, rc, max_context)


@pytest.mark.parametrize("quality", [0, 1, 2])
@pytest.mark.parametrize("block", [1, 2, 4, 7])
def test_every_drafter_quality_reproduces_the_sequential_stream(oracle, quality, block):
    # crates/runtime/tests/speculative.rs:597 — greedy speculative == greedy sequential
    e1, t1, em1, r1, _ = _scripted(oracle, quality, 0, 0, block=block)
    e2, t2, em2, r2, c2 = _scripted(oracle, quality, 0, 1, block=block)
    assert e1 == 0 and e2 == 0
    assert np.array_equal(t1, t2) and np.array_equal(em1, em2)
    assert r1.new_tokens == r2.new_tokens == 64 and r1.reason == r2.reason == 0
    assert r2.kv_position == r2.history_len
    if quality == 0:
        assert r2.accepted_total >= r2.rounds  # a perfect drafter is accepted
    if quality == 1:
        assert r2.accepted_total == 0 and c2[1] == r2.rollbacks > 0  # retaining rollback is what runs


def test_budget_window_and_admission(oracle):
    # exact budget (:747), never feeds past the window (:779), refusals (raw_completion.rs:126-146)
    e, t, em, r, c = _scripted(oracle, 0, 0, 1, block=4, max_new=10)
    assert e == 0 and r.new_tokens == 10 and len(em) == 10
    e, t, em, r, c = _scripted(oracle, 0, 0, 1, block=7, max_new=20, prompt_len=5, max_context=25)
    assert e == 0 and c[4] < 25
    assert _scripted(oracle, 0, 0, 1, block=0)[0] == -4
    assert _scripted(oracle, 0, 0, 1, max_new=0)[0] == -2
    assert _scripted(oracle, 0, 0, 1, prompt_len=0)[0] == -1
    assert _scripted(oracle, 0, 0, 1, max_new=30, max_context=32)[0] == -3


def test_stop_token_inside_an_accepted_block(oracle):
    # crates/runtime/tests/speculative.rs:711
    e, t, em, r, _ = _scripted(oracle, 0, 0, 0, block=4, max_new=64)
    stop_tok = int(em[6])
    e1, t1, em1, r1, _ = _scripted(oracle, 0, 0, 0, block=4, stop=(stop_tok,))
    e2, t2, em2, r2, _ = _scripted(oracle, 0, 0, 1, block=4, stop=(stop_tok,))
    assert r1.reason == r2.reason == 1
    assert np.array_equal(em1, em2) and np.array_equal(t1, t2)
    assert em2[-1] == stop_tok and t2[-1] != stop_tok or len(t2) == len(em2) + 5 - 1


def test_sampled_speculative_matches_sequential_in_distribution(oracle):
    # crates/runtime/tests/speculative.rs:870-1000 — TV distance over seeds, graded three-way target
    vocab = 97
    for quality in (0, 1, 2):
        counts_seq = np.zeros(vocab)
        counts_spec = np.zeros(vocab)
        n = 600
        for seed in range(n):
            _, _, em1, _, _ = _scripted(oracle, quality, 1, 0, temperature=0.7, max_new=4, seed=seed)
            _, _, em2, _, _ = _scripted(oracle, quality, 1, 1, temperature=0.7, max_new=4, seed=seed + 100000, block=3)
            counts_seq[em1[1]] += 1
            counts_spec[em2[1]] += 1
        tv = 0.5 * np.abs(counts_seq / n - counts_spec / n).sum()
        assert tv < 0.08, (quality, tv)


def test_adaptive_depth_controller(oracle):
    # crates/runtime/src/speculative_adaptive.rs:104-225
    import ctypes as C
    a = oracle.Adaptive()
    L = oracle.lib()
    L.tso_adaptive_init(C.byref(a), C.c_int64(2), C.c_int64(5))
    assert a.cur == 2
    for _ in range(7):
        L.tso_adaptive_observe(C.byref(a), C.c_int64(2), C.c_int64(2))
    assert a.cur == 2
    L.tso_adaptive_observe(C.byref(a), C.c_int64(2), C.c_int64(2))
    assert a.cur == 3
    L.tso_adaptive_observe(C.byref(a), C.c_int64(3), C.c_int64(2))
    assert a.cur == 3 and a.pressure == 1
    L.tso_adaptive_observe(C.byref(a), C.c_int64(3), C.c_int64(2))
    assert a.cur == 2 and a.pressure == 0
    L.tso_adaptive_observe(C.byref(a), C.c_int64(2), C.c_int64(0))
    assert a.cur == 2  # never below the floor
    assert L.tso_adaptive_tile_cap(15, 8) == 7 and L.tso_adaptive_tile_cap(15, -1) == 15 and L.tso_adaptive_tile_cap(15, 1) == 1


def test_tree_spec_paths_and_walk(oracle):
    # crates/runtime/src/families/qwen/batched_scratch.rs:97-124, crates/runtime/src/dflash_tree.rs
    import json, os
    parent = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "tree_parent.json")))["parent"]
    depth, paths = oracle.tree_spec(parent)
    assert list(depth) == [0, 1, 2, 3, 4, 1, 2, 3]
    assert list(paths[7][:4]) == [0, 1, 2, 7] and list(paths[6][:3]) == [0, 5, 6]
    with pytest.raises(ValueError):
        oracle.tree_spec([-1, 2, 1])
    with pytest.raises(ValueError):
        oracle.tree_spec([0, 0])
    assert list(oracle.tree_slot_parents([-1, 0, -1, 1])) == [-1, 0, 1, 0, 2]
    # best-first: parents precede children, the spine is greedy (dflash_tree.rs tests)
    scores = np.tile(-np.arange(4, dtype=np.float32), (4, 1))
    scores[0, 1] = -0.2
    d, c, p = oracle.best_first_tree(scores, 7)
    assert len(d) == 7 and (d[0], c[0]) == (0, 0) and (d[1], c[1]) == (0, 1)
    for i in range(7):
        if p[i] >= 0:
            assert p[i] < i and d[p[i]] + 1 == d[i]
    # acceptance walk
    node_parent = [-1, -1, 0, 0, 2]
    node_token = [10, 11, 20, 21, 30]
    pick = [10, 20, 0, 30, 0, 99]  # per slot: anchor->10, slot1->20, slot3->30, slot5->99
    assert list(oracle.tree_accept(node_parent, node_token, pick)) == [0, 2, 4]


def test_gather_rows_refuses_non_compactions(oracle):
    # crates/gpu/src/dflash_conv.rs:192-234
    rows = np.arange(8 * 4, dtype=np.uint16).reshape(8, 4).copy()
    want = rows[[0, 2, 5]].copy()
    assert oracle.gather_rows_inplace(rows, [0, 2, 5]) == 0
    assert np.array_equal(rows[:3], want)
    assert oracle.gather_rows_inplace(rows, [1, 0]) == 1
    assert oracle.gather_rows_inplace(rows, [0, 2, 2]) == 1


def test_moe_routing_follows_the_router_rules(oracle):
    """router_topk_gemma4 (crates/runtime/src/real_forward_dispatch.rs:1135-1158): top-k by logit, ties to the lower
    index, softmax over the selected logits only, times the per-expert scale."""
    lg = np.array([[0.5, 2.0, -1.0, 2.0, 1.0, 0.0]], dtype=np.float32)
    ids, w = oracle.moe_route(lg, 3)
    assert ids.tolist() == [[1, 3, 4]]
    e = np.exp(np.array([0.0, 0.0, -1.0], dtype=np.float32))
    want = (e / e.sum()).astype(np.float32)
    assert np.allclose(oracle.f16_bits_to_f32(w[0]), want, rtol=1e-3)
    # not a softmax over all experts: the weights of the selected ones sum to one
    assert abs(float(oracle.f16_bits_to_f32(w[0]).sum()) - 1.0) < 2e-3
    ids2, w2 = oracle.moe_route(lg, 3, scale=np.array([1, 2, 1, 0.5, 1, 1], dtype=np.float32))
    assert ids2.tolist() == [[1, 3, 4]]
    assert np.allclose(oracle.f16_bits_to_f32(w2[0]), want * np.array([2, 0.5, 1], dtype=np.float32), rtol=1e-3)
