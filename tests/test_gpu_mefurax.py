"""Mefurax on the GPU against the plain oracle (tests/mefurax_oracle.py): every mechanism alone, prompts against token-by-token
decoding, portions, unequal batches, slot reuse, window and chunk edges, far keys, odd sizes, greedy generation through the scheduler.

The library runs in its f32 compute mode where the comparison has to be sharp (errors ~1e-6) and in bf16 mode with a bound that a
wrong mechanism exceeds by orders of magnitude."""
import copy

import numpy as np
import pytest

import mefurax_oracle as O
import mefurax_synth as S

pytestmark = pytest.mark.gpu

F32_TOL = 2e-4
BF16_TOL = 6e-2


def tokens(n, vocab, seed=1):
    return [int(t) for t in np.random.default_rng(seed).integers(0, vocab, n)]


def check_whole(cfg, n, seed=0, compute="float32", tol=F32_TOL, taps=True, w=None):
    w = w if w is not None else S.random_weights(cfg, seed)
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
                assert np.abs(gt[r] - rt[r]).max() <= tol * np.abs(rt[r]).max() * 4, f"residual stream after layer {r}"
        assert S.rel_err(got, want) < tol
    finally:
        gpu.close()
    return want


# ---------------------------------------------------------------------------------------------------- mechanisms alone
def test_windowed_mixer_alone(b200):
    # biases, convolution, whole-projection norm, distance bias, window shorter than the prompt; no feed-forward, no value sharing
    check_whole(S.config([S.layer_a(v_mix=False)]), 40)


def test_chunked_mixer_alone(b200):
    # rotation on part of the head, unit norm per head, soft cap, chunks shorter than the prompt, one gate per head
    check_whole(S.config([S.layer_b(v_mix=False)]), 40)


def test_soft_cap_bites(b200):
    # scores far above the cap: without the tanh the softmax would be one-hot
    cfg = S.config([S.layer_b(v_mix=False, softcap=1.5, scale=4.0, chunk=16)])
    want = check_whole(cfg, 33, seed=2)
    loose = copy.deepcopy(cfg)
    loose["layers"][0]["mixer"]["softcap"] = 50.0
    other = O.Model(loose, S.random_weights(cfg, 2)).forward(tokens(33, cfg["vocab"], 3))
    assert S.rel_err(other[5:], want[5:]) > 50 * F32_TOL


def test_gated_gelu_feed_forward(b200):
    check_whole(S.config([S.layer_b(v_mix=False, mlp=S.dense(88))]), 24, seed=3)


def test_mixture_of_experts(b200):
    check_whole(S.config([S.layer_a(v_mix=False, mlp=S.moe(experts=6, top=3, ff=24, shared=40))]), 30, seed=4)


def test_mixture_without_always_on_expert_and_single_choice(b200):
    check_whole(S.config([S.layer_b(v_mix=False, mlp=S.moe(experts=3, top=1, ff=20, shared=0)),
                          S.layer_a(v_mix=False, mlp=S.moe(experts=4, top=4, ff=12, shared=8))]), 26, seed=5)


def test_router_choice_is_the_largest_logits(b200):
    # the router's rows are made of one-hot directions times distinct gains, so the order of the logits is known; expert 2's down
    # projection is blown up: a model that picked it when it should not (or missed it) would be far off
    cfg = S.config([S.layer_b(v_mix=False, mlp=S.moe(experts=5, top=2, ff=16, shared=0))], width=48)
    w = S.random_weights(cfg, 6)
    w["l0.mlp.e2.down"] = w["l0.mlp.e2.down"] * 8
    check_whole(cfg, 40, seed=6, w=w)


@pytest.mark.parametrize("order", ["ab", "ba", "aab"])
def test_values_shared_across_layers(b200, order):
    # the first marked layer is the source whatever its kind; an unmarked layer in between neither reads nor replaces it
    kinds = {"a": S.layer_a, "b": S.layer_b}
    layers = [kinds[c](v_mix=True, mlp=S.dense(40) if i == 0 else None) for i, c in enumerate(order)]
    layers.insert(1, S.layer_b(v_mix=False, heads=2, kv_heads=1, dim=16, vdim=24))
    cfg = S.config(layers)
    want = check_whole(cfg, 28, seed=7)
    off = copy.deepcopy(cfg)
    for L in off["layers"]:
        L["mixer"]["v_mix"] = False
    assert S.rel_err(O.Model(off, S.random_weights(cfg, 7)).forward(tokens(28, cfg["vocab"], 8)), want) > 50 * F32_TOL


def full_cfg():
    return S.config([S.layer_b(mlp=S.dense(72)), S.layer_a(window=6, conv=4, mlp=S.moe()), S.layer_b(chunk=5, mlp=S.moe(experts=4, top=2, ff=16, shared=0)),
                     S.layer_a(window=11, conv=2, mlp=None)])


def test_whole_model(b200):
    check_whole(full_cfg(), 45, seed=9)


def test_bf16_mode_whole_model(b200):
    check_whole(full_cfg(), 48, seed=10, compute="bfloat16", tol=BF16_TOL, taps=False)


# ---------------------------------------------------------------------------------------------------- other sizes
@pytest.mark.parametrize("layers,width,alpha", [
    # one head, sizes that are not multiples of 4 / 8 / 32, a window and a chunk of one position, one tap, rotation of the whole head
    ([S.layer_a(heads=1, kv_heads=1, dim=10, vdim=14, window=1, conv=1, mlp=S.dense(20)),
      S.layer_b(heads=1, kv_heads=1, dim=10, vdim=14, chunk=1, rot_dims=10, mlp=S.moe(experts=2, top=1, ff=6, shared=10))], 36, 1.0),
    # wide heads (keys above 128, values above 128), one K/V head for all query heads, no rotation, no cap, a long filter, window and chunk
    # longer than the prompt
    ([S.layer_b(heads=4, kv_heads=1, dim=136, vdim=72, chunk=300, rot_dims=0, softcap=0.0, mlp=None),
      S.layer_a(heads=3, kv_heads=3, dim=72, vdim=24, window=300, conv=6, mlp=S.dense(96))], 104, 3.0),
    # key and value sizes equal, every head its own K/V head, no convolution at all
    ([S.layer_a(heads=6, kv_heads=6, dim=32, vdim=32, conv=0, mlp=S.moe(experts=9, top=4, ff=32, shared=32)),
      S.layer_b(heads=6, kv_heads=6, dim=32, vdim=32, rot_dims=32, mlp=S.dense(64))], 64, 0.5),
])
def test_other_sizes(b200, layers, width, alpha):
    cfg = S.config(layers, width=width, vocab=70, eps=1e-6, alpha=alpha)
    check_whole(cfg, 27, seed=11)


# ---------------------------------------------------------------------------------------------------- schedules
def test_prompt_against_token_by_token(b200):
    cfg = full_cfg()
    w = S.random_weights(cfg, 13)
    toks = tokens(34, cfg["vocab"], 14)
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
    # the filter's tail, the chunk count and the window all have to carry over the cuts
    cfg = full_cfg()
    w = S.random_weights(cfg, 15)
    toks = tokens(37, cfg["vocab"], 16)
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
    cfg = full_cfg()
    w = S.random_weights(cfg, 17)
    ref = O.Model(cfg, w)
    prompts = [tokens(n, cfg["vocab"], 20 + n) for n in (1, 13, 29, 6)]
    tails = [tokens(9, cfg["vocab"], 40 + i) for i in range(4)]
    gpu = S.gpu_model(cfg, w, max_batch=6)
    try:
        slots = [4, 0, 2, 5]
        got = gpu.step(list(zip(slots, prompts)), list(range(sum(len(p) for p in prompts))))
        at, states = 0, []
        for p in prompts:
            st = ref.new_state()
            assert S.rel_err(got[at:at + len(p)], ref.step(st, p)) < F32_TOL
            states.append(st)
            at += len(p)
        for k in range(9):                                          # the shortest request ends first, then the next one
            alive = [i for i in range(4) if k < 3 + 2 * i]
            lg = gpu.decode_batch([slots[i] for i in alive], [tails[i][k] for i in alive])
            for j, i in enumerate(alive):
                assert S.rel_err(lg[j], ref.step(states[i], [tails[i][k]])[0]) < F32_TOL, (k, i)
    finally:
        gpu.close()


def test_bf16_batch_rows_do_not_depend_on_the_batch(b200):
    cfg = S.config([S.layer_b(dim=32, mlp=S.dense(72)), S.layer_a(dim=32, window=20, mlp=S.moe())])
    w = S.random_weights(cfg, 18)
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
    cfg = full_cfg()
    w = S.random_weights(cfg, 19)
    ref = O.Model(cfg, w)
    gpu = S.gpu_model(cfg, w, max_batch=3)
    try:
        assert gpu.pool_counts() == (0, 0)
        a, b, c = tokens(30, cfg["vocab"], 3), tokens(18, cfg["vocab"], 4), tokens(25, cfg["vocab"], 5)
        gpu.step([(0, a), (1, b)])
        assert gpu.pool_counts() == (2, 0)
        gpu.reset(0)
        assert gpu.pool_counts() == (1, 1) and gpu.position(0) == 0
        # slot 2 takes the block that slot 0 left (full of a's keys and filter tail); slot 1 goes on undisturbed
        got = gpu.step([(2, c)], list(range(len(c))))
        assert gpu.pool_counts() == (2, 0)
        assert S.rel_err(got, ref.forward(c)) < F32_TOL
        st = ref.new_state()
        ref.step(st, b)
        for t in tokens(5, cfg["vocab"], 6):
            assert S.rel_err(gpu.forward(t, seq=1), ref.step(st, [t])[0]) < F32_TOL
        gpu.reset(2)
        gpu.reset(1)
        got = gpu.step([(1, a)], [len(a) - 1])
        assert S.rel_err(got, ref.forward(a)[-1]) < F32_TOL
    finally:
        gpu.close()


# ---------------------------------------------------------------------------------------------------- window and chunk edges
def edge_cfg(kind, size):
    # one mixer alone with scores of order one: every visible key carries a few percent of the weight, so one key more or less in
    # view moves the logits far beyond the tolerance.  Head 0's distance slope would drown far keys; the scale keeps them alive.
    if kind == "window":
        return S.config([S.layer_a(heads=2, kv_heads=1, dim=16, vdim=24, window=size, conv=2, scale=1.0, v_mix=False)], width=48, vocab=64)
    return S.config([S.layer_b(heads=2, kv_heads=1, dim=16, vdim=24, chunk=size, rot_dims=8, softcap=20.0, scale=1.0, v_mix=False)], width=48, vocab=64)


@pytest.mark.parametrize("kind", ["window", "chunk"])
@pytest.mark.parametrize("decode", [False, True])
def test_mask_edges(b200, kind, decode):
    size = 11
    cfg = edge_cfg(kind, size)
    w = S.random_weights(cfg, 21)
    n = 64
    toks = tokens(n, cfg["vocab"], 22)
    want = O.Model(cfg, w).forward(toks)
    # the oracle itself must tell the neighbouring masks apart at most positions, or the test would prove nothing
    for other in (size - 1, size + 1):
        alt_cfg = copy.deepcopy(cfg)
        alt_cfg["layers"][0]["mixer"]["mask"]["size"] = other
        alt = O.Model(alt_cfg, w).forward(toks)
        far = [p for p in range(size + 2, n) if S.rel_err(alt[p], want[p]) > 20 * F32_TOL]
        assert len(far) > (n - size) // 2, other
    gpu = S.gpu_model(cfg, w)
    try:
        if decode:
            gpu.step([(0, toks[:3])])
            for p in range(3, n):
                assert S.rel_err(gpu.forward(toks[p]), want[p]) < F32_TOL, p
        else:
            got = gpu.step([(0, toks)], list(range(n)))
            for p in range(n):
                assert S.rel_err(got[p], want[p]) < F32_TOL, p
    finally:
        gpu.close()


def test_chunks_count_from_the_sequence_start_not_from_the_cut(b200):
    # a prompt cut in the middle of a chunk: the second portion's first tokens still see the first portion's last ones, and nothing else
    cfg = edge_cfg("chunk", 8)
    w = S.random_weights(cfg, 23)
    toks = tokens(40, cfg["vocab"], 24)
    want = O.Model(cfg, w).forward(toks)
    gpu = S.gpu_model(cfg, w)
    try:
        a = gpu.step([(0, toks[:13])], list(range(13)))
        b = gpu.step([(0, toks[13:])], list(range(27)))
        assert S.rel_err(np.concatenate([a, b]), want) < F32_TOL
    finally:
        gpu.close()


@pytest.mark.parametrize("kind", ["window", "chunk"])
def test_far_key_among_hundreds(b200, kind):
    # position 300 still sees position 8.  The embedding row of the probe token (positions 296 on) is solved for, so that its query is
    # a multiple of the needle token's key (position 8) in every head: that one score stands out among hundreds of random ones, also
    # against the distance bias of the windowed mixer (2^-8 per position for the last head).
    size = 296 if kind == "window" else 320
    cfg = edge_cfg(kind, size)
    m = cfg["layers"][0]["mixer"]
    if kind == "window":
        m["conv"], m["scale"] = 0, 4.0
    else:                           # (unit heads of 16 channels: an aligned pair scores 16, a random one about +-4)
        m["softcap"], m["scale"] = 60.0, 1.0
    w = S.random_weights(cfg, 25)
    if kind == "window":
        for n_ in ("q", "k", "v"):
            w["l0.mix.%s.b" % n_] = 0 * w["l0.mix.%s.b" % n_]
    n = 310
    toks = tokens(n, cfg["vocab"] - 2, 26)
    needle, probe = cfg["vocab"] - 2, cfg["vocab"] - 1
    k_needle = (w["l0.mix.k"].astype(np.float64) @ w["embed"][needle]).reshape(m["kv_heads"], m["dim"])
    if kind == "chunk":             # rotated keys: the probe's query at position 301 meets the needle's key of position 8
        k_needle = np.stack([O.rotate_pairs(r, 301 - 8, m["rot"]["dims"], m["rot"]["base"]) for r in k_needle])
    target = np.concatenate([k_needle[h // (m["heads"] // m["kv_heads"])] for h in range(m["heads"])])
    e = np.linalg.pinv(w["l0.mix.q"].astype(np.float64)) @ target
    w["embed"][probe] = S.bf16_to_f32(S.bf16_bits((e * (np.linalg.norm(w["embed"][needle]) / np.linalg.norm(e))).astype(np.float32)))
    toks[8] = needle
    for p in range(296, n):
        toks[p] = probe
    ref = O.Model(cfg, w)
    want = ref.forward(toks)
    gpu = S.gpu_model(cfg, w, max_seq_len=n + 4)
    try:
        got = gpu.step([(0, toks[:300])], list(range(290, 300)))
        assert S.rel_err(got, want[290:300]) < F32_TOL
        for p in range(300, n):
            assert S.rel_err(gpu.forward(toks[p]), want[p]) < F32_TOL, p
    finally:
        gpu.close()
    # with the needle replaced the answers at the far end change: the far key is really seen, in the prompt and in decoding
    toks2 = list(toks)
    toks2[8] = 0
    alt = ref.forward(toks2)
    for p in (299, 300, 301):
        assert S.rel_err(alt[p], want[p]) > 40 * F32_TOL, p
    if kind == "window":            # and position 8 has left the window of position 304
        assert S.rel_err(alt[304:], want[304:]) < 1e-9


def test_first_tokens_and_long_decoding(b200):
    cfg = full_cfg()
    w = S.random_weights(cfg, 27)
    toks = tokens(120, cfg["vocab"], 28)      # more than ten windows and chunks decoded one by one, from the very first token
    ref = O.Model(cfg, w)
    st = ref.new_state()
    gpu = S.gpu_model(cfg, w)
    try:
        for p, t in enumerate(toks):
            assert S.rel_err(gpu.forward(t), ref.step(st, [t])[0]) < F32_TOL, p
    finally:
        gpu.close()


def test_rotation_at_large_positions(b200):
    # angles in the thousands of radians: an f32 angle would already be off in the fourth digit
    cfg = S.config([S.layer_b(heads=2, kv_heads=2, dim=16, vdim=16, chunk=2048, rot_dims=16, rot_base=4.0, softcap=0.0, scale=1.5, v_mix=False)],
                   width=32, vocab=40)
    w = S.random_weights(cfg, 29)
    n = 1500
    toks = tokens(n, cfg["vocab"], 30)
    ref = O.Model(cfg, w)
    st = ref.new_state()
    # the oracle only has to attend at the last positions; earlier tokens just fill its lists
    gpu = S.gpu_model(cfg, w, max_seq_len=n + 4)
    try:
        got = gpu.step([(0, toks)], [n - 2, n - 1])
        want = ref.step(st, toks)[-2:]
        assert S.rel_err(got, want) < F32_TOL
    finally:
        gpu.close()


# ---------------------------------------------------------------------------------------------------- the scheduler
def test_greedy_generation_through_the_batched_engine(b200):
    cfg = full_cfg()
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
    cfg = full_cfg()
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
    cfg = S.config([S.layer_a(v_mix=False)])
    w = S.random_weights(cfg, 41)
    gpu = S.gpu_model(cfg, w, max_seq_len=16)
    try:
        with pytest.raises(b200.InvalidArgument):
            gpu.step([(0, [cfg["vocab"]])])
        with pytest.raises(b200.InvalidArgument):
            gpu.step([(0, tokens(17, cfg["vocab"]))])
        assert gpu.path() == "layers"
    finally:
        gpu.close()
    del w["l0.mix.q.conv"]
    with pytest.raises(b200.InvalidArgument):
        S.gpu_model(cfg, w)
    # values blended from a source of another size
    bad = S.config([S.layer_a(vdim=40), S.layer_b(vdim=24)])
    with pytest.raises(b200.InvalidArgument):
        S.gpu_model(bad, S.random_weights(bad, 42))


# ---------------------------------------------------------------------------------------------------- kernels against their plain forms
@pytest.mark.parametrize("kind,dims", [("window", (16, 24, 11)), ("window", (32, 40, 70)), ("chunk", (96, 56, 23)), ("chunk", (128, 128, 64)),
                                       ("window", (64, 40, 64))])
def test_tile_attention_against_warp_attention(b200, monkeypatch, kind, dims):
    # bf16 prompts take the tensor-pipe attention kernel when the head sizes allow it; the warp kernel computes the same thing in f32.
    # Windows and chunks that end inside, at and across key tiles of 64; several unequal runs in one step, one of them continued
    # afterwards (its cache then holds rows of both steps, and its chunks go on counting from its own start).
    dim, vdim, size = dims
    if kind == "window":
        cfg = S.config([S.layer_a(heads=4, kv_heads=2, dim=dim, vdim=vdim, window=size, v_mix=False)], width=64, vocab=80)
    else:
        cfg = S.config([S.layer_b(heads=4, kv_heads=2, dim=dim, vdim=vdim, chunk=size, rot_dims=16, v_mix=False)], width=64, vocab=80)
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
    bm = ref.forward(b + more)
    want = np.concatenate([ref.forward(a), bm[:len(b)], ref.forward(c), bm[len(b):]])
    assert S.rel_err(outs["1"], outs["0"]) < 2e-2
    assert S.rel_err(outs["1"], want) < BF16_TOL
    assert S.rel_err(outs["0"], want) < BF16_TOL


def test_tensor_core_gemm_path(b200, monkeypatch):
    # bf16 mode with enough rows for the tcgen05 GEMM (fused [gate | up], the experts' wide product, K that is not a multiple of 64)
    # against the CUDA-core kernel on the same operands
    cfg = S.config([S.layer_b(heads=4, kv_heads=2, dim=32, vdim=40, chunk=50, mlp=S.dense(200)),
                    S.layer_a(heads=4, kv_heads=2, dim=32, vdim=40, window=60, conv=4, mlp=S.moe(experts=6, top=2, ff=40, shared=24))], width=168, vocab=300)
    w = S.random_weights(cfg, 43)
    toks = tokens(300, cfg["vocab"], 44)
    outs = {}
    for tc in ("1", "0"):
        monkeypatch.setenv("B200_LP_TC", tc)
        gpu = S.gpu_model(cfg, w, "bfloat16", max_seq_len=320)
        try:
            rows = [gpu.step([(0, toks[:n])], list(range(n))) for n in (40, 100)]
            gpu.reset(0)
            rows.append(gpu.step([(1, toks)], list(range(300))))
            outs[tc] = rows
        finally:
            gpu.close()
    # (a router logit that the two summation orders put on different sides of a neighbour flips an expert: rows are compared in bulk)
    for a, b in zip(outs["1"], outs["0"]):
        d = np.array([S.rel_err(a[i], b[i]) for i in range(len(a))])
        assert np.median(d) < 1.5e-2 and (d < 1.5e-2).mean() > 0.9
    ref = O.Model(cfg, w).forward(toks)
    d = np.array([S.rel_err(outs["1"][2][i], ref[i]) for i in range(300)])
    assert np.median(d) < BF16_TOL and (d < BF16_TOL).mean() > 0.9


# ---------------------------------------------------------------------------------------------------- the command line
def test_trace_runner_on_a_model_folder(b200, tmp_path):
    # config.json + model.safetensors (bf16) on disk -> registry -> bin/trace_run: two requests start together with unequal prompts, are
    # decoded together, the shorter one ends first; logits of the wanted rows come back in files
    import json
    import os
    import subprocess
    import sys

    from llama_gguf_b200.safetensors_io import bf16_bits, write_safetensors

    cfg = full_cfg()
    w = S.random_weights(cfg, 51)
    d = tmp_path / "model"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(cfg))
    write_safetensors(str(d / "model.safetensors"), {n: bf16_bits(a).reshape(a.shape) for n, a in w.items()})
    a, b = tokens(19, cfg["vocab"], 52), tokens(7, cfg["vocab"], 53)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": a[:15], "want": [0, 14]}, {"id": "y", "tokens": b[:5], "want": [4]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": a[15:16], "want": []}, {"id": "y", "tokens": b[5:6], "want": [0]}], "end": []},
             {"step": 2, "entries": [{"id": "x", "tokens": a[16:17], "want": [0]}, {"id": "y", "tokens": b[6:7], "want": [0]}], "end": ["y"]},
             {"step": 3, "entries": [{"id": "x", "tokens": a[17:19], "want": [1]}], "end": ["x"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(d), "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [ln for ln in r.stdout.split("\n") if ln.startswith("done")] == ["done %d" % i for i in range(4)]
    ref = O.Model(cfg, w)
    wa, wb = ref.forward(a), ref.forward(b)
    got = {i: np.fromfile(str(out / ("%d.f32" % i)), dtype="<f4").reshape(-1, cfg["vocab"]) for i in range(4)}
    assert S.rel_err(got[0], np.stack([wa[0], wa[14], wb[4]])) < F32_TOL
    assert S.rel_err(got[1], wb[5:6]) < F32_TOL
    assert S.rel_err(got[2], np.stack([wa[16], wb[6]])) < F32_TOL
    assert S.rel_err(got[3], wa[18:19]) < F32_TOL


def test_decode_kernels_for_few_rows_against_the_many_row_path(b200, monkeypatch):
    # decoding reads only the chosen experts' weights (a kernel per projection that walks the router's picks); B200_LP_FUSE=0 sends
    # the same rows through the products over all experts.  Both against the oracle, in a batch whose members sit at different
    # positions, in f32; and against each other in bf16.
    cfg = S.config([S.layer_b(mlp=S.moe(experts=6, top=2, ff=24, shared=16)), S.layer_a(conv=4, mlp=S.moe(experts=3, top=3, ff=8, shared=0)),
                    S.layer_b(chunk=4, mlp=S.moe(experts=4, top=1, ff=32, shared=8))])
    w = S.random_weights(cfg, 53)
    ref = O.Model(cfg, w)
    prompts = [tokens(n, cfg["vocab"], 60 + n) for n in (3, 19, 1)]
    tails = [tokens(12, cfg["vocab"], 70 + i) for i in range(3)]
    states = [ref.new_state() for _ in prompts]
    for st, pr in zip(states, prompts):
        ref.step(st, pr)
    want = [[ref.step(states[i], [tails[i][k]])[0] for i in range(3)] for k in range(12)]
    bf = {}
    for fuse in ("1", "0"):
        monkeypatch.setenv("B200_LP_FUSE", fuse)
        for compute in ("float32", "bfloat16"):
            gpu = S.gpu_model(cfg, w, compute)
            try:
                gpu.step([(i, pr) for i, pr in enumerate(prompts)])
                rows = []
                for k in range(12):
                    lg = gpu.decode_batch([0, 1, 2], [tails[i][k] for i in range(3)])
                    rows.append(lg)
                    if compute == "float32":
                        for i in range(3):
                            assert S.rel_err(lg[i], want[k][i]) < F32_TOL, (fuse, k, i)
                if compute == "bfloat16":
                    bf[fuse] = np.concatenate(rows)
            finally:
                gpu.close()
    d = np.array([S.rel_err(bf["1"][i], bf["0"][i]) for i in range(len(bf["1"]))])
    assert np.median(d) < 2e-2 and (d < 2e-2).mean() > 0.9
