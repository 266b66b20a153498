"""Lazilorn on the GPU against the plain oracle (tests/lazilorn_oracle.py): every mechanism alone, prompts against token-by-token
decoding, portions, unequal batches, slot reuse, window and kept-first edges, odd sizes, greedy generation through the scheduler.

The library runs in its f32 compute mode where the comparison has to be sharp (errors ~1e-6) and in bf16 mode once per family
with a bound that a wrong mechanism exceeds by orders of magnitude."""
import numpy as np
import pytest

import lazilorn_oracle as O
import lazilorn_synth as S

pytestmark = pytest.mark.gpu

F32_TOL = 2e-4
BF16_TOL = 6e-2


def tokens(n, vocab, seed=1):
    return [int(t) for t in np.random.default_rng(seed).integers(0, vocab, n)]


def check_whole(cfg, n, seed=0, compute="float32", tol=F32_TOL, taps=True):
    w = S.random_weights(cfg, seed)
    ref = O.Model(cfg, w)
    toks = tokens(n, cfg["vocab"], seed + 1)
    rt = []
    want = ref.forward(toks, rt)
    gpu = S.gpu_model(cfg, w, compute, max_seq_len=n + 8, taps=taps)
    try:
        got = gpu.step([(0, toks)], list(range(n)))
        if taps:
            gt = gpu.taps(n)
            assert gt.shape[0] == len(rt)
            for r in range(len(rt)):
                scale = np.abs(rt[r]).max()
                assert np.abs(gt[r] - rt[r]).max() <= tol * scale * 4, f"residual stream after layer run {r}"
        assert S.rel_err(got, want) < tol
    finally:
        gpu.close()
    return want


# ---------------------------------------------------------------------------------------------------- mechanisms alone
def test_embedding_and_attention_alone(b200):
    # right_scale = 0 silences the matrix memory; window and kept tokens smaller than the prompt
    cfg = S.config([S.parallel_layer(left_scale=1.0, right_scale=0.0, ff=0)])
    check_whole(cfg, 40)


def test_matrix_memory_alone(b200):
    cfg = S.config([S.parallel_layer(left_scale=0.0, right_scale=1.0, ff=0, mheads=3, mdim=16, mvdim=40)])
    check_whole(cfg, 40)


def test_gated_delta_alone(b200):
    cfg = S.config([S.delta_layer(ff=0)])
    check_whole(cfg, 40)


def test_feed_forward_and_layer_without_one(b200):
    cfg = S.config([S.delta_layer(ff=72), S.delta_layer(ff=0)])
    check_whole(cfg, 24)


def test_repeated_range_with_step_vectors(b200):
    # three passes over layers 1..2, each on a state of its own; layer 0 before and layer 3 after run once
    cfg = S.config([S.delta_layer(ff=48), S.parallel_layer(), S.delta_layer(heads=2, kv_heads=2), S.parallel_layer(ff=0)], loop=(1, 3, 3))
    w = S.random_weights(cfg, 3)
    assert O.Model(cfg, w).runs == [0, 1, 2, 1, 2, 1, 2, 3]
    check_whole(cfg, 30, seed=3)


def test_bf16_mode_whole_model(b200):
    cfg = S.config([S.parallel_layer(), S.delta_layer(ff=64), S.parallel_layer(window=5, keep_first=2)], loop=(0, 2, 2))
    check_whole(cfg, 48, compute="bfloat16", tol=BF16_TOL, taps=False)


# ---------------------------------------------------------------------------------------------------- other sizes
@pytest.mark.parametrize("layers,width,loop", [
    # sizes that are not multiples of 4 / 8 / 32, one head, equal head counts, a window of one, no kept tokens, one tap
    ([S.parallel_layer(heads=1, kv_heads=1, dim=10, vdim=14, window=1, keep_first=0, mheads=1, mdim=6, mvdim=10, ff=20),
      S.delta_layer(heads=1, kv_heads=1, dim=6, vdim=10, conv=1, ff=0)], 36, (0, 0, 1)),
    # wide heads: key size above 64 and value size above 128, kept tokens longer than the window, long convolution
    ([S.parallel_layer(heads=4, kv_heads=4, dim=72, vdim=136, window=4, keep_first=9, mheads=1, mdim=80, mvdim=72, ff=96),
      S.delta_layer(heads=2, kv_heads=1, dim=136, vdim=72, conv=6, ff=40)], 104, (1, 2, 2)),
    # repeated range that is the whole model, run once (times = 1: the step vector still counts)
    ([S.delta_layer(heads=6, kv_heads=2, dim=32, vdim=32, conv=2), S.parallel_layer(heads=6, kv_heads=2, dim=32, vdim=32)], 64, (0, 2, 1)),
])
def test_other_sizes(b200, layers, width, loop):
    cfg = S.config(layers, width=width, vocab=70, loop=loop, eps=1e-6, embed_scale=1.5, logit_scale=1.3)
    check_whole(cfg, 27, seed=5)


# ---------------------------------------------------------------------------------------------------- schedules
def mixed_cfg():
    return S.config([S.parallel_layer(window=6, keep_first=2), S.delta_layer(conv=4, ff=56), S.parallel_layer(window=9, keep_first=0, ff=0)],
                    loop=(1, 3, 2))


def test_prompt_against_token_by_token(b200):
    cfg = mixed_cfg()
    w = S.random_weights(cfg, 7)
    toks = tokens(34, cfg["vocab"], 8)
    want = O.Model(cfg, w).forward(toks)
    gpu = S.gpu_model(cfg, w)
    try:
        rows = [gpu.forward(t) for t in toks]                       # every token decoded alone, from the first one
        assert S.rel_err(np.stack(rows), want) < F32_TOL
        assert gpu.position() == len(toks)
        gpu.reset()
        last = gpu.forward_batch(toks[:20])                         # prompt, then decoding
        assert S.rel_err(last, want[19]) < F32_TOL
        for p in range(20, len(toks)):
            assert S.rel_err(gpu.forward(toks[p]), want[p]) < F32_TOL, p
    finally:
        gpu.close()


@pytest.mark.parametrize("portion", [2, 3, 7, 16])
def test_portions(b200, portion):
    cfg = mixed_cfg()
    w = S.random_weights(cfg, 9)
    toks = tokens(37, cfg["vocab"], 10)
    want = O.Model(cfg, w).forward(toks)
    gpu = S.gpu_model(cfg, w)
    try:
        got = []
        for a in range(0, len(toks), portion):
            part = toks[a:a + portion]
            got.append(gpu.step([(1, part)], list(range(len(part)))))
        assert S.rel_err(np.concatenate(got), want) < F32_TOL
    finally:
        gpu.close()


def test_unequal_batch_against_each_alone(b200):
    cfg = mixed_cfg()
    w = S.random_weights(cfg, 11)
    ref = O.Model(cfg, w)
    prompts = [tokens(n, cfg["vocab"], 20 + n) for n in (1, 13, 29, 6)]
    tails = [tokens(9, cfg["vocab"], 40 + i) for i in range(4)]
    gpu = S.gpu_model(cfg, w, max_batch=6)
    try:
        slots = [4, 0, 2, 5]
        runs = [(s, p) for s, p in zip(slots, prompts)]
        rows = list(range(sum(len(p) for p in prompts)))
        got = gpu.step(runs, rows)
        at = 0
        states = []
        for p in prompts:
            st = ref.new_state()
            want = ref.step(st, p)
            states.append(st)
            assert S.rel_err(got[at:at + len(p)], want) < F32_TOL
            at += len(p)
        # decode together; the shortest request ends first, then the next one
        for k in range(9):
            alive = [i for i in range(4) if k < 3 + 2 * i]
            lg = gpu.decode_batch([slots[i] for i in alive], [tails[i][k] for i in alive])
            for j, i in enumerate(alive):
                want = ref.step(states[i], [tails[i][k]])
                assert S.rel_err(lg[j], want[0]) < F32_TOL, (k, i)
    finally:
        gpu.close()


def test_bf16_batch_rows_do_not_depend_on_the_batch(b200):
    cfg = mixed_cfg()
    w = S.random_weights(cfg, 12)
    a, b = tokens(21, cfg["vocab"], 1), tokens(40, cfg["vocab"], 2)
    gpu = S.gpu_model(cfg, w, "bfloat16")
    try:
        alone = gpu.step([(0, a)], list(range(len(a))))
        both = gpu.step([(1, b), (2, a)], list(range(len(b), len(b) + len(a))))
        assert S.rel_err(both, alone) < 2e-2
        assert S.rel_err(alone, O.Model(cfg, w).forward(a)) < BF16_TOL
    finally:
        gpu.close()


def test_slots_freed_and_used_again(b200):
    cfg = mixed_cfg()
    w = S.random_weights(cfg, 13)
    ref = O.Model(cfg, w)
    gpu = S.gpu_model(cfg, w, max_batch=3)
    try:
        assert gpu.pool_counts() == (0, 0)
        a, b, c = tokens(30, cfg["vocab"], 3), tokens(18, cfg["vocab"], 4), tokens(25, cfg["vocab"], 5)
        gpu.step([(0, a), (1, b)])
        assert gpu.pool_counts() == (2, 0)
        gpu.reset(0)
        assert gpu.pool_counts() == (1, 1) and gpu.position(0) == 0
        # slot 2 takes the block that slot 0 left (full of a's keys and state); slot 1 goes on undisturbed
        got = gpu.step([(2, c)], list(range(len(c))))
        assert gpu.pool_counts() == (2, 0)
        assert S.rel_err(got, ref.forward(c)) < F32_TOL
        nxt = tokens(5, cfg["vocab"], 6)
        st = ref.new_state()
        ref.step(st, b)
        for t in nxt:
            assert S.rel_err(gpu.forward(t, seq=1), ref.step(st, [t])[0]) < F32_TOL
        # both blocks back in the pool, one of them taken again
        gpu.reset(2)
        gpu.reset(1)
        got = gpu.step([(1, a)], [len(a) - 1])
        assert S.rel_err(got, ref.forward(a)[-1]) < F32_TOL
        with pytest.raises(b200.InvalidArgument):
            gpu.step([(0, a), (0, b)])
    finally:
        gpu.close()


# ---------------------------------------------------------------------------------------------------- window edges
def attention_only_cfg(window, keep_first):
    # attention alone with scores of order one: every visible key carries a few percent of the weight, so one key more or less
    # in view moves the logits far beyond the tolerance
    return S.config([S.parallel_layer(heads=2, kv_heads=1, dim=16, vdim=24, window=window, keep_first=keep_first,
                                      left_scale=1.0, right_scale=0.0, ff=0)], width=48, vocab=64)


def variant(cfg, window, keep_first):
    import copy
    c = copy.deepcopy(cfg)
    c["layers"][0]["mixer"]["left"]["mask"] = {"size": window, "keep_first": keep_first}
    return c


@pytest.mark.parametrize("decode", [False, True])
def test_window_and_kept_first_edges(b200, decode):
    window, keep = 11, 4
    cfg = attention_only_cfg(window, keep)
    w = S.random_weights(cfg, 17)
    n = 64
    toks = tokens(n, cfg["vocab"], 18)
    want = O.Model(cfg, w).forward(toks)
    # the oracle itself must tell the neighbouring masks apart at most positions, or the test would prove nothing
    for other in ((window - 1, keep), (window + 1, keep), (window, keep - 1), (window, keep + 1)):
        alt = O.Model(variant(cfg, *other), w).forward(toks)
        far = [p for p in range(window + keep + 2, n) if S.rel_err(alt[p], want[p]) > 20 * F32_TOL]
        assert len(far) > (n - window - keep) // 2, other
    gpu = S.gpu_model(cfg, w)
    try:
        if decode:
            gpu.step([(0, toks[:3])])
            got = np.stack([gpu.forward(t) for t in toks[3:]])
            for p in range(3, n):
                assert S.rel_err(got[p - 3], want[p]) < F32_TOL, p
        else:
            got = gpu.step([(0, toks)], list(range(n)))
            for p in range(n):
                assert S.rel_err(got[p], want[p]) < F32_TOL, p
    finally:
        gpu.close()


def test_far_key_among_hundreds(b200):
    # a wide window: position 300 still sees position 8 (and kept token 1); a needle key that only one far query matches
    cfg = S.config([S.parallel_layer(heads=2, kv_heads=2, dim=16, vdim=24, window=296, keep_first=2, scale=6.0,
                                     left_scale=1.0, right_scale=0.0, ff=0)], width=48, vocab=64)
    w = S.random_weights(cfg, 19)
    n = 310
    toks = tokens(n, cfg["vocab"], 20)
    ref = O.Model(cfg, w)
    want = ref.forward(toks)
    gpu = S.gpu_model(cfg, w, max_seq_len=n + 4)
    try:
        got = gpu.step([(0, toks[:290])], list(range(280, 290)))
        assert S.rel_err(got, want[280:290]) < F32_TOL
        for p in range(290, n):
            assert S.rel_err(gpu.forward(toks[p]), want[p]) < F32_TOL, p
    finally:
        gpu.close()


def test_first_tokens_and_long_decoding(b200):
    cfg = mixed_cfg()
    w = S.random_weights(cfg, 23)
    toks = tokens(120, cfg["vocab"], 24)      # more than ten windows decoded one by one, from the very first token
    ref = O.Model(cfg, w)
    st = ref.new_state()
    gpu = S.gpu_model(cfg, w)
    try:
        for p, t in enumerate(toks):
            assert S.rel_err(gpu.forward(t), ref.step(st, [t])[0]) < F32_TOL, p
    finally:
        gpu.close()


def test_matrix_memory_gates_at_their_caps(b200):
    # large gate pre-activations: the soft cap and the running maximum do the work
    cfg = S.config([S.parallel_layer(left_scale=0.0, right_scale=1.0, ff=0, cap=4.0)])
    w = S.random_weights(cfg, 29)
    w["l0.mix.right.i"] = w["l0.mix.right.i"] * 16
    w["l0.mix.right.f"] = w["l0.mix.right.f"] * 16
    toks = tokens(50, cfg["vocab"], 30)
    want = O.Model(cfg, w).forward(toks)
    gpu = S.gpu_model(cfg, w)
    try:
        assert S.rel_err(gpu.step([(0, toks)], list(range(50))), want) < F32_TOL
    finally:
        gpu.close()


# ---------------------------------------------------------------------------------------------------- the scheduler
def test_greedy_generation_through_the_batched_engine(b200):
    cfg = mixed_cfg()
    w = S.random_weights(cfg, 31)
    ref = O.Model(cfg, w)
    prompts = [tokens(n, cfg["vocab"], 50 + n) for n in (5, 17, 9, 26, 3)]
    n_new = [6, 4, 8, 5, 7]
    want = []
    for p, k in zip(prompts, n_new):
        st = ref.new_state()
        lg = ref.step(st, p)[-1]
        out = []
        for _ in range(k):
            t = int(len(lg) - 1 - np.argmax(lg[::-1]))      # last maximum wins
            out.append(t)
            lg = ref.step(st, [t])[0]
        want.append(out)
    gpu = S.gpu_model(cfg, w, max_batch=3)
    eng = b200.BatchedEngine(gpu, max_batch_size=3, max_seq_len=200, eos_token_id=cfg["vocab"] + 7)   # (no token is EOS)
    try:
        ids = [eng.submit(p, k) for p, k in zip(prompts, n_new)]   # five requests on three slots: two wait, slots are reused
        got = {i: [] for i in ids}
        done = {}
        for ev in eng.run():
            if ev[0] == "token":
                got[ev[1]].append(ev[2])
            elif ev[0] == "done":
                done[ev[1]] = ev[2:]
            else:
                raise AssertionError(ev)
        for i, rid in enumerate(ids):
            assert got[rid] == want[i], i
            assert done[rid] == ("max_tokens", len(prompts[i]), n_new[i])
        assert gpu.pool_counts()[0] <= 3
    finally:
        eng.close()
        gpu.close()


def test_decode_greedy_entry_point(b200):
    cfg = mixed_cfg()
    w = S.random_weights(cfg, 37)
    ref = O.Model(cfg, w)
    p = tokens(12, cfg["vocab"], 38)
    st = ref.new_state()
    ref.step(st, p[:-1])
    gpu = S.gpu_model(cfg, w)
    try:
        gpu.step([(0, p[:-1])])
        out, _ = gpu.decode_greedy(p[-1], 6)
        t, want = p[-1], []
        for _ in range(6):
            lg = ref.step(st, [t])[0]
            t = int(len(lg) - 1 - np.argmax(lg[::-1]))
            want.append(t)
        assert out.tolist() == want
    finally:
        gpu.close()


def test_bad_arguments(b200):
    cfg = S.config([S.delta_layer()])
    w = S.random_weights(cfg, 41)
    gpu = S.gpu_model(cfg, w, max_seq_len=16)
    try:
        with pytest.raises(b200.InvalidArgument):
            gpu.step([(0, [cfg["vocab"]])])
        with pytest.raises(b200.InvalidArgument):
            gpu.step([(0, tokens(17, cfg["vocab"]))])
        with pytest.raises(b200.InvalidArgument):
            gpu.step([(9, [1])])
        assert gpu.path() == "layers"
    finally:
        gpu.close()
    del w["l0.mix.A_log"]
    with pytest.raises(b200.InvalidArgument):
        S.gpu_model(cfg, w)


# ---------------------------------------------------------------------------------------------------- tensor-core GEMM
def test_tensor_core_gemm_against_cuda_core_gemm(b200, monkeypatch):
    # bf16 mode, sizes that reach every tile width of the tcgen05 kernel (rows 40 / 100 / 300), a K that is not a multiple of 64,
    # output widths that are not multiples of 128; the CUDA-core kernel multiplies the same bf16 values, so the two paths differ
    # only in the order of the f32 sums (and in the bf16 roundings of later activations that such a difference flips)
    cfg = S.config([S.parallel_layer(heads=4, kv_heads=2, dim=32, vdim=40, window=50, keep_first=3, mheads=3, mdim=32, mvdim=40, ff=200),
                    S.delta_layer(heads=4, kv_heads=2, dim=32, vdim=48, conv=4, ff=136)], width=168, vocab=300)
    w = S.random_weights(cfg, 43)
    toks = tokens(300, cfg["vocab"], 44)
    outs = {}
    for tc in ("1", "0"):
        monkeypatch.setenv("B200_LP_TC", tc)
        gpu = S.gpu_model(cfg, w, "bfloat16", max_seq_len=320)
        try:
            rows = [gpu.step([(0, toks[:n])], list(range(n))) for n in (40, 100)]
            gpu.reset(0)
            gpu.reset(1)
            rows.append(gpu.step([(1, toks)], list(range(300))))
            outs[tc] = rows
        finally:
            gpu.close()
    for a, b in zip(outs["1"], outs["0"]):
        assert S.rel_err(a, b) < 1.5e-2
    assert S.rel_err(outs["1"][2], O.Model(cfg, w).forward(toks)) < BF16_TOL


@pytest.mark.parametrize("dims", [(16, 24, 11, 4), (32, 40, 70, 0), (96, 136, 23, 30), (128, 128, 64, 1)])
def test_tile_attention_against_warp_attention(b200, monkeypatch, dims):
    # bf16 prompts take the tensor-pipe attention kernel when the head sizes allow it; the warp kernel computes the same thing in
    # f32.  Windows that end inside, at and across key tiles of 64; kept tokens shorter and longer than the window; several unequal
    # runs in one step, one of them continued afterwards (its cache then holds rows of both steps).
    dim, vdim, window, keep = dims
    cfg = S.config([S.parallel_layer(heads=4, kv_heads=2, dim=dim, vdim=vdim, window=window, keep_first=keep, left_scale=1.0,
                                     right_scale=0.0, ff=0)], width=64, vocab=80)
    w = S.random_weights(cfg, 47)
    a, b, c = tokens(150, cfg["vocab"], 1), tokens(64, cfg["vocab"], 2), tokens(17, cfg["vocab"], 3)
    more = tokens(70, cfg["vocab"], 4)
    outs = {}
    for tile in ("1", "0"):
        monkeypatch.setenv("B200_LP_ATTN_TILE", tile)
        gpu = S.gpu_model(cfg, w, "bfloat16", max_seq_len=256)
        try:
            first = gpu.step([(0, a), (1, b), (2, c)], list(range(len(a) + len(b) + len(c))))
            second = gpu.step([(1, more)], list(range(len(more))))
            outs[tile] = np.concatenate([first, second])
        finally:
            gpu.close()
    ref = O.Model(cfg, w)
    want = np.concatenate([ref.forward(a), ref.forward(b + more)[:len(b)], ref.forward(c), ref.forward(b + more)[len(b):]])
    assert S.rel_err(outs["1"], outs["0"]) < 2e-2
    assert S.rel_err(outs["1"], want) < BF16_TOL
    assert S.rel_err(outs["0"], want) < BF16_TOL


def test_fused_decode_kernels_against_unfused(b200, monkeypatch):
    # decoding takes fused kernels (norm inside the projection, q/k norm and the cache write inside attention, the convolution
    # tail moved on by the convolution itself); B200_LP_FUSE=0 runs every step as its own kernel.  Both against the oracle, in a
    # batch whose members sit at different positions, f32 mode.
    cfg = S.config([S.parallel_layer(heads=4, kv_heads=2, dim=24, vdim=40, window=7, keep_first=2), S.delta_layer(conv=4, ff=56),
                    S.parallel_layer(heads=2, kv_heads=2, dim=16, vdim=24, window=30, keep_first=0, ff=0)], loop=(0, 2, 2))
    w = S.random_weights(cfg, 53)
    ref = O.Model(cfg, w)
    prompts = [tokens(n, cfg["vocab"], 60 + n) for n in (3, 19, 1)]
    tails = [tokens(12, cfg["vocab"], 70 + i) for i in range(3)]
    states = [ref.new_state() for _ in prompts]
    for st, pr in zip(states, prompts):
        ref.step(st, pr)
    want = [[ref.step(states[i], [tails[i][k]])[0] for i in range(3)] for k in range(12)]
    for fuse in ("1", "0"):
        monkeypatch.setenv("B200_LP_FUSE", fuse)
        gpu = S.gpu_model(cfg, w)
        try:
            gpu.step([(i, pr) for i, pr in enumerate(prompts)])
            for k in range(12):
                lg = gpu.decode_batch([0, 1, 2], [tails[i][k] for i in range(3)])
                for i in range(3):
                    assert S.rel_err(lg[i], want[k][i]) < F32_TOL, (fuse, k, i)
        finally:
            gpu.close()
