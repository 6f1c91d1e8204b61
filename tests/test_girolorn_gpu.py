"""The Girolorn design in the engine against the plain float64 oracle (oracle/girolorn.py): every mechanism alone, whole
prompts against pieces and token-by-token decoding, mixed batches, reused pages and slots, far keys and page borders with
peaked scores, sinks and caps that bite, the first tokens, long decoding, other sizes, layers that share tensors, and
greedy generation through the scheduler.  float32 engines give the sharp comparison; bfloat16 ones are held to a
rounding-sized bound."""
import copy

import numpy as np
import pytest
import torch

from oracle import girolorn as og

pytestmark = pytest.mark.gpu


def make_engine(kge, tmp_path, cfg, W, dtype="float32", tokens=512, bs=16, seqs=4, name="m", batched=0):
    d = str(tmp_path / name)
    og.save_model_dir(d, cfg, W)
    nb = (tokens + bs - 1) // bs
    return kge.LLM(d, dtype=dtype, block_size=bs, num_gpu_blocks_override=nb + 1, max_model_len=nb * bs + 1, max_num_seqs=seqs,
                   max_num_batched_tokens=batched or nb * bs, enable_prefix_caching=False)


def run_pieces(llm, rid, tokens, pieces):
    """Feed `tokens` in steps of the given sizes, asking for every position's logits."""
    out, at = [], 0
    for n in pieces:
        llm.trace_add(rid, tokens[at:at + n])
        out.append(llm.trace_step([(rid, n, list(range(n)))]))
        at += n
    assert at == len(tokens)
    return np.concatenate(out)


def check(got, want, dtype, what="", margins=None):
    """Row-wise error against the oracle, relative to the logits' size.  bfloat16 engines form the router's logits from
    rounded activations: where the oracle's own choice hangs on a margin below 0.05 (`margins`, per token) another expert
    may be chosen, so such rows are left out, and the rows after the first of them, which see that token through the
    attention of later layers, get a wider bound (still far below what a lost key, a wrong position or a wrong expert
    weight costs: 0.3 and more).  The float32 runs of the same cases are the sharp ones."""
    want = want.numpy() if isinstance(want, torch.Tensor) else want
    scale = np.sqrt((want ** 2).mean())
    err = np.sqrt(((got - want) ** 2).mean(-1)) / scale
    lim = np.full(len(err), 2e-4 if dtype == "float32" else 4e-2)
    if dtype != "float32" and margins is not None:
        close = np.asarray(margins) < 0.05
        assert close.mean() < 0.5, f"{what}: {close.sum()} of {len(close)} rows hang on a close routing call"
        if close.any():
            lim[int(np.argmax(close)):] = 0.15
            lim[close] = np.inf
    worst = int(np.argmax(err / lim))
    assert (err < lim).all(), f"{what}: row {worst} is {err[worst]:.3g} of the logits' size (limit {lim[worst]:.3g})"


def oracle(cfg, W, toks):
    """Logits and routing margins as numpy arrays."""
    lg, mg = og.forward(cfg, W, toks, return_margins=True)
    return lg.numpy(), mg.numpy()


def prompt(cfg, n, seed=1):
    return torch.randint(0, cfg["vocab"], (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def silence_attention(W):
    for k in W:
        if k.endswith("mix.o"):
            W[k] = torch.zeros_like(W[k])
    return W


ALONE = {
    "attention": dict(n_layers=1, mlps=(False,)),
    "attention-plain-frequencies": dict(n_layers=1, mlps=(False,), scaling=None),
    "attention-no-rotation": dict(n_layers=1, mlps=(False,), rot_dims=0),
    "attention-all-dims-rotate": dict(n_layers=1, mlps=(False,), rot_dims=12),
    "attention-no-cap": dict(n_layers=1, mlps=(False,), softcap=0.0, logit_softcap=0.0),
    "attention-one-kv-head": dict(n_layers=1, mlps=(False,), kv_heads=1),
    "moe": dict(n_layers=1),
    "moe-noshared": dict(n_layers=1, shared=False, top=3),
    "moe-top1": dict(n_layers=1, top=1),
    "moe-all-experts": dict(n_layers=1, experts=3, top=3),
}


@pytest.mark.parametrize("mech", sorted(ALONE))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mechanism_alone(kge, tmp_path, mech, dtype):
    cfg = og.make_config(**ALONE[mech])
    W = og.make_weights(cfg, seed=3)
    if mech.startswith("moe"):
        silence_attention(W)
    toks = prompt(cfg, 45)
    llm = make_engine(kge, tmp_path, cfg, W, dtype)
    got = run_pieces(llm, 0, toks, [45])
    llm.close()
    want, mg = oracle(cfg, W, toks)
    check(got, want, dtype, mech, mg)


FULL = dict(n_layers=4, weights_of={2: 0, 3: 1}, mlps=(True, True, True, True))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_decode_and_pieces_agree_with_the_oracle(kge, tmp_path, dtype):
    cfg = og.make_config(**FULL)
    W = og.make_weights(cfg, seed=5)
    toks = prompt(cfg, 75)
    want, mg = oracle(cfg, W, toks)
    llm = make_engine(kge, tmp_path, cfg, W, dtype)
    for rid, pieces in enumerate([[75], [30] + [1] * 45, [1] * 75, [2, 3, 17, 2, 31, 5, 2, 2, 9, 2], [23, 2, 24, 26], [47, 2, 1, 1, 24]]):
        got = run_pieces(llm, rid, toks, pieces)
        llm.trace_end(rid)
        check(got, want, dtype, f"pieces {pieces[:6]}", mg)
    llm.close()


def test_layer_outputs_match(kge, tmp_path):
    """The residual stream after every layer run; layers 2 and 3 run with the tensors of 0 and 1 and caches of their own."""
    cfg = og.make_config(**FULL)
    W = og.make_weights(cfg, seed=6)
    toks = prompt(cfg, 33)
    _, layers = og.forward(cfg, W, toks, return_layers=True)
    llm = make_engine(kge, tmp_path, cfg, W, "float32")
    buf = np.zeros((4, 33, cfg["width"]), dtype=np.float32)
    llm.set_layer_dump(buf)
    run_pieces(llm, 0, toks, [33])
    llm.set_layer_dump(None)
    llm.close()
    for i, x in enumerate(layers):
        assert np.abs(buf[i] - x.numpy()).max() < 2e-4 * float(x.abs().max()), f"layer {i}"


def test_shared_tensors_keep_their_own_cache(kge, tmp_path):
    """A model whose second layer runs with the first layer's tensors differs from a one-layer model, and decoding it
    token by token (each layer reading its own cache) equals the whole prompt."""
    cfg = og.make_config(n_layers=2, weights_of={1: 0})
    W = og.make_weights(cfg, seed=21)
    toks = prompt(cfg, 40, 5)
    want = og.forward(cfg, W, toks)
    one = og.forward(og.make_config(n_layers=1), W, toks)
    assert float((want - one).abs().max()) > 0.1
    llm = make_engine(kge, tmp_path, cfg, W, "float32")
    check(run_pieces(llm, 0, toks, [10] + [1] * 30), want, "float32")
    llm.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_of_unequal_requests(kge, tmp_path, dtype):
    cfg = og.make_config(**FULL)
    W = og.make_weights(cfg, seed=7)
    P = {0: prompt(cfg, 61, 10), 1: prompt(cfg, 9, 11), 2: prompt(cfg, 40, 12), 3: prompt(cfg, 1, 13)}
    want = {r: oracle(cfg, W, t) for r, t in P.items()}
    # each step: (request, number of tokens); prompt pieces beside single tokens, requests pausing and resuming
    steps = [[(0, 19), (1, 1), (3, 1)], [(1, 1), (2, 2), (0, 2)], [(0, 20), (1, 1)], [(2, 18), (1, 1), (0, 1)], [(1, 5), (2, 1)],
             [(0, 1), (2, 1)], [(0, 18), (2, 18)]]
    llm = make_engine(kge, tmp_path, cfg, W, dtype)
    at = {r: 0 for r in P}
    got = {r: [] for r in P}
    for st in steps:
        entries = []
        for r, n in st:
            llm.trace_add(r, P[r][at[r]:at[r] + n])
            entries.append((r, n, list(range(n))))
        lg = llm.trace_step(entries)
        k = 0
        for r, n in st:
            got[r].append(lg[k:k + n])
            k += n
            at[r] += n
    llm.close()
    for r in P:
        assert at[r] == len(P[r])
        check(np.concatenate(got[r]), want[r][0], dtype, f"request {r}", want[r][1])


def test_pages_and_slots_are_used_again(kge, tmp_path):
    """Two request slots and a pool of 96 tokens: five requests pass through, each in pages that an earlier request
    filled; each must come out as if it had run alone."""
    cfg = og.make_config(**FULL)
    W = og.make_weights(cfg, seed=8)
    llm = make_engine(kge, tmp_path, cfg, W, "float32", tokens=96, bs=16, seqs=2)
    P = {r: prompt(cfg, n, 20 + r) for r, n in enumerate([40, 33, 47, 18, 30])}
    want = {r: og.forward(cfg, W, t).numpy() for r, t in P.items()}
    got = {}
    got[0] = run_pieces(llm, 0, P[0], [40])
    llm.trace_add(1, P[1][:20])
    a = llm.trace_step([(1, 20, list(range(20)))])
    llm.trace_end(0)
    llm.trace_add(2, P[2])
    llm.trace_add(1, P[1][20:])
    b = llm.trace_step([(2, 30, list(range(30))), (1, 13, list(range(13)))])
    got[1] = np.concatenate([a, b[30:]])
    c = llm.trace_step([(2, 17, list(range(17)))])
    got[2] = np.concatenate([b[:30], c])
    llm.trace_end(1)
    got[3] = run_pieces(llm, 3, P[3], [2, 16])
    llm.trace_end(2)
    llm.trace_end(3)
    got[4] = run_pieces(llm, 4, P[4], [29, 1])
    llm.close()
    for r in P:
        check(got[r], want[r], "float32", f"request {r}")


def peaked(dim, **kw):
    """Attention alone with scores that reach the cap: single keys carry most of a row's weight, so a key that is lost,
    misplaced in its page or rotated by the wrong position moves the logits far beyond rounding; sinks of real weight."""
    return og.make_config(n_layers=1, mlps=(False,), dim=dim, rot_dims=dim - 4, scale=4.0, softcap=12.0, **kw)


@pytest.mark.parametrize("dim", [12, 32])        # the per-row kernel; the tensor-core kernel (bfloat16, key size a multiple of 16)
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_far_keys_and_page_borders_with_peaked_scores(kge, tmp_path, dtype, dim):
    cfg = peaked(dim, heads=4, kv_heads=2)
    W = og.make_weights(cfg, seed=9)
    toks = prompt(cfg, 330, 30)
    want = og.forward(cfg, W, toks)
    # the setup shows what it should: without the first page's keys, or without the sinks, late rows move visibly
    late = og.forward(cfg, W, toks[16:])[-30:]
    assert float((late - want[-30:]).abs().max()) > 0.2
    nosink = dict(W)
    nosink["l0.mix.sink"] = torch.full_like(W["l0.mix.sink"], -50.0)
    assert float((og.forward(cfg, nosink, toks[:40]) - want[:40]).abs().max()) > 0.2
    llm = make_engine(kge, tmp_path, cfg, W, dtype, bs=16)
    check(run_pieces(llm, 0, toks, [330]), want, dtype, "whole")
    llm.trace_end(0)
    check(run_pieces(llm, 1, toks[:100], [15, 1, 1, 1, 14, 2, 30, 1, 1, 34]), want[:100], dtype, "pieces and single tokens across page borders")
    llm.trace_end(1)
    got = np.concatenate([run_pieces(llm, 2, toks[:290], [290]), run_pieces(llm, 2, toks[290:], [1] * 40)])
    check(got, want, dtype, "decoding far from the first keys")
    llm.close()


def test_sinks_decide_short_rows(kge, tmp_path):
    """Large sinks: the first rows give most of their weight to the sink, so the mixer's output is scaled down by a
    factor that only the sink explains; per head different."""
    cfg = og.make_config(n_layers=1, mlps=(False,), heads=3, kv_heads=3, dim=16, rot_dims=16, softcap=3.0)
    W = og.make_weights(cfg, seed=19)
    W["l0.mix.sink"] = torch.tensor([4.0, -3.0, 1.5], dtype=og.DT)
    toks = prompt(cfg, 24, 3)
    want = og.forward(cfg, W, toks)
    for dtype in ("float32", "bfloat16"):
        llm = make_engine(kge, tmp_path, cfg, W, dtype, name=dtype)
        check(run_pieces(llm, 0, toks, [1, 1, 2, 20]), want, dtype, dtype)
        llm.close()


def test_long_prompt_tensor_core_kernels(kge, tmp_path):
    """bfloat16 at sizes the tensor-core paths take: 64-wide heads, grouped heads, 64-token pages, several key tiles per
    warp, prompts long enough for the 64-row attention CTAs."""
    cfg = og.make_config(n_layers=2, width=64, heads=4, kv_heads=2, dim=64, rot_dims=32, scale=0.5, softcap=9.0, experts=4, expert_ff=64, shared_ff=64,
                         weights_of={1: 0})
    W = og.make_weights(cfg, seed=15)
    toks = prompt(cfg, 290, 32)
    want, mg = oracle(cfg, W, toks)
    llm = make_engine(kge, tmp_path, cfg, W, "bfloat16", bs=64)
    got = np.concatenate([run_pieces(llm, 0, toks[:150], [150]), run_pieces(llm, 0, toks[150:260], [3, 45, 2, 60]), run_pieces(llm, 0, toks[260:], [1] * 30)])
    llm.close()
    check(got, want, "bfloat16", "", mg)


@pytest.mark.parametrize("shape", [(4, 4, 128, 64), (6, 2, 64, 64), (8, 1, 64, 32), (2, 1, 128, 128), (5, 1, 64, 16)])
def test_tensor_core_head_sizes(kge, tmp_path, shape):
    """bfloat16, 64-token pages, attention alone with scores at the cap and sinks of real weight, at the head sizes and
    group sizes (1, 2, 3, 5 and 8 query heads per key/value head) that the tcgen05 prompt kernel and the TMA-staged decode
    kernels take; prompt steps, pieces beside nothing else, decoding over a page border, a decode batch of unequal
    contexts, and single tokens beside a prompt piece in one step."""
    heads, kv, dim, rot = shape
    cfg = og.make_config(n_layers=2, width=64, heads=heads, kv_heads=kv, dim=dim, rot_dims=rot, scale=1.4 * (12 / dim) ** 0.5, softcap=10.0,
                         mlps=(False, False), weights_of={1: 0})
    W = og.make_weights(cfg, seed=23)
    W["l0.mix.sink"] = torch.linspace(-1.0, 3.0, heads, dtype=og.DT)
    toks = prompt(cfg, 230, 34)
    want = og.forward(cfg, W, toks)
    nosink = dict(W)
    nosink["l0.mix.sink"] = torch.full_like(W["l0.mix.sink"], -50.0)
    assert float((og.forward(cfg, nosink, toks[:30]) - want[:30]).abs().max()) > 0.2
    llm = make_engine(kge, tmp_path, cfg, W, "bfloat16", bs=64, tokens=1024)
    check(run_pieces(llm, 0, toks, [230]), want, "bfloat16", "whole")
    llm.trace_end(0)
    got = np.concatenate([run_pieces(llm, 1, toks[:180], [61, 3, 2, 64, 50]), run_pieces(llm, 1, toks[180:], [1] * 50)])
    check(got, want, "bfloat16", "pieces, then decoding")
    # two requests decoding side by side (one far longer than the other) and a third that brings a prompt piece
    a, b = prompt(cfg, 150, 35), prompt(cfg, 9, 36)
    wa, wb = og.forward(cfg, W, a).numpy(), og.forward(cfg, W, b).numpy()
    llm.trace_add(2, a[:140])
    llm.trace_add(3, b[:3])
    llm.trace_step([(2, 140, []), (3, 3, [])])
    ga, gb = [], []
    for i in range(6):
        llm.trace_add(2, a[140 + i:141 + i])
        llm.trace_add(3, b[3 + i:4 + i])
        lg = llm.trace_step([(2, 1, [0]), (3, 1, [0])])
        ga.append(lg[0])
        gb.append(lg[1])
    # one more token of the long request beside the first piece of a new prompt and a lone first token
    c, d1 = prompt(cfg, 70, 37), prompt(cfg, 1, 38)
    llm.trace_end(3)
    llm.trace_add(2, a[146:147])
    llm.trace_add(4, c[:66])
    llm.trace_add(5, d1)
    lg = llm.trace_step([(2, 1, [0]), (4, 66, list(range(66))), (5, 1, [0])])
    llm.close()
    check(np.stack(ga), wa[140:146], "bfloat16", "long request of a decode batch")
    check(np.stack(gb), wb[3:9], "bfloat16", "short request of a decode batch")
    check(lg[:1], wa[146:147], "bfloat16", "a single token beside a prompt piece")
    check(lg[1:67], og.forward(cfg, W, c).numpy()[:66], "bfloat16", "a prompt piece beside single tokens")
    check(lg[67:], og.forward(cfg, W, d1).numpy(), "bfloat16", "a lone first token in a mixed step")


def test_experts_with_many_routed_rows(kge, tmp_path):
    """A prompt long enough that the routed rows are made contiguous per expert and run as one tensor-core GEMM pair per
    expert (bfloat16; expert width a multiple of 64); the same prompt fed in short pieces takes the grouped kernel.
    Limits small enough that the clamps cut a good part of the pre-activations."""
    cfg = og.make_config(n_layers=1, width=64, experts=6, top=2, expert_ff=64, shared_ff=128, expert_limit=0.4, shared_limit=0.3)
    W = silence_attention(og.make_weights(cfg, seed=16))
    toks = prompt(cfg, 300, 33)
    want, mg = oracle(cfg, W, toks)
    loose = copy.deepcopy(cfg)
    loose["layers"][0]["mlp"]["expert"]["limit"] = 50.0
    assert float(np.abs(og.forward(loose, W, toks).numpy() - want).max()) > 0.1
    llm = make_engine(kge, tmp_path, cfg, W, "bfloat16", bs=64)
    check(run_pieces(llm, 0, toks, [300]), want, "bfloat16", "one step", mg)
    llm.trace_end(0)
    check(run_pieces(llm, 1, toks, [280, 7, 13]), want, "bfloat16", "pieces", mg)
    llm.close()


def test_first_tokens(kge, tmp_path):
    cfg = og.make_config(**FULL)
    W = og.make_weights(cfg, seed=11)
    llm = make_engine(kge, tmp_path, cfg, W, "float32")
    for rid, n in enumerate([1, 2, 3, 5]):
        toks = prompt(cfg, n, 40 + n)
        got = run_pieces(llm, rid, toks, [n])
        llm.trace_end(rid)
        check(got, og.forward(cfg, W, toks), "float32", f"{n} tokens")
    llm.close()


def test_long_decoding(kge, tmp_path):
    cfg = og.make_config(**FULL)
    W = og.make_weights(cfg, seed=12)
    toks = prompt(cfg, 200, 50)
    llm = make_engine(kge, tmp_path, cfg, W, "float32")
    got = run_pieces(llm, 0, toks, [4] + [1] * 196)
    llm.close()
    check(got, og.forward(cfg, W, toks), "float32")


@pytest.mark.parametrize("sizes", [
    dict(n_layers=2, heads=3, kv_heads=3, dim=16, rot_dims=16, experts=2, top=1, scaling=(2.0, 16, 4.0, 1.0)),
    dict(n_layers=3, vocab=53, width=40, heads=6, kv_heads=2, dim=10, rot_dims=6, base=300.0, scaling=(16.0, 24, 3.0, 0.25), scale=0.9, softcap=2.5,
         experts=9, top=4, expert_ff=11, expert_limit=0.6, shared_ff=13, shared_limit=3.0, mlps=(True, False, True), weights_of={2: 0}, eps=1e-3,
         logit_softcap=3.0),
    dict(n_layers=1, heads=2, kv_heads=1, dim=7, rot_dims=4, expert_ff=5, shared=False),
    dict(n_layers=2, vocab=67, width=42, heads=3, kv_heads=1, dim=14, rot_dims=10, experts=3, top=2, expert_ff=64, shared_ff=64),      # rows of 84 bytes: nothing is 16-byte aligned
    dict(n_layers=2, vocab=72, width=44, heads=2, kv_heads=2, dim=16, rot_dims=16, experts=4, top=3, expert_ff=24, shared_ff=8, weights_of={1: 0}),
])
def test_other_sizes(kge, tmp_path, sizes):
    cfg = og.make_config(**sizes)
    W = og.make_weights(cfg, seed=13)
    toks = prompt(cfg, 50, 60)
    want, mg = oracle(cfg, W, toks)
    llm = make_engine(kge, tmp_path, cfg, W, "float32")
    check(run_pieces(llm, 0, toks, [50]), want, "float32", "whole")
    check(run_pieces(llm, 1, toks, [13, 2, 1, 1, 1, 32]), want, "float32", "pieces")
    llm.close()
    llm = make_engine(kge, tmp_path, cfg, W, "bfloat16", name="b")        # the same sizes through the 16-bit kernels and their fallbacks
    check(run_pieces(llm, 0, toks, [50]), want, "bfloat16", "whole, bfloat16", mg)
    check(run_pieces(llm, 1, toks, [13, 2, 1, 1, 1, 32]), want, "bfloat16", "pieces, bfloat16", mg)
    llm.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_scheduler(kge, tmp_path, dtype):
    """LLM.generate: the continuous-batching scheduler cuts the prompts into 16-token steps, admits the third request
    when a slot frees up, and samples greedily."""
    cfg = og.make_config(**FULL)
    W = og.make_weights(cfg, seed=14)
    prompts = [prompt(cfg, n, 70 + n) for n in (37, 5, 21)]
    llm = make_engine(kge, tmp_path, cfg, W, dtype, seqs=2, batched=16)
    outs = llm.generate(prompts, kge.SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True))
    assert llm.kernel_launches > 0
    llm.close()
    for p, o in zip(prompts, outs):
        got = o.outputs[0].token_ids
        assert len(got) == 12
        toks = list(p)
        for k, g in enumerate(got):       # teacher-forced: a different choice must be a near-tie of the oracle
            lg = og.forward(cfg, W, toks)[-1]
            best = int(torch.argmax(lg))
            if g != best:      # the samplers read 16-bit logits rows: two logits within their spacing tie
                gap = float(lg[best] - lg[g])
                assert gap < (2.0 ** -7 * max(1.0, float(lg[best].abs())) if dtype == "float32" else 0.15), f"token {k}: chose {g}, oracle {best} leads by {gap}"
            toks.append(g)


def test_greedy_generation_with_decode_graphs(kge, tmp_path):
    """LLM.generate at a head size the TMA-staged decode kernels take (bfloat16, 64-token pages): after the prompts the
    decode steps are captured as a CUDA graph and replayed while the contexts grow over a page border; every sampled token
    must be the oracle's choice or a near-tie of it."""
    cfg = og.make_config(n_layers=2, width=64, heads=4, kv_heads=2, dim=64, rot_dims=32, scale=0.35, softcap=9.0, experts=4, top=2, expert_ff=64,
                         shared_ff=64, weights_of={1: 0})
    W = og.make_weights(cfg, seed=24)
    prompts = [prompt(cfg, n, 90 + n) for n in (57, 9)]
    llm = make_engine(kge, tmp_path, cfg, W, "bfloat16", bs=64, tokens=512, seqs=2, batched=64)
    outs = llm.generate(prompts, kge.SamplingParams(max_tokens=20, temperature=0.0, ignore_eos=True))
    llm.close()
    for p, o in zip(prompts, outs):
        got = o.outputs[0].token_ids
        assert len(got) == 20
        toks = list(p)
        for k, g in enumerate(got):
            lg = og.forward(cfg, W, toks)[-1]
            best = int(torch.argmax(lg))
            if g != best:
                gap = float(lg[best] - lg[g])
                assert gap < 0.2, f"token {k}: chose {g}, oracle {best} leads by {gap}"
            toks.append(g)


def test_trace_runner_command_line(kge, tmp_path):
    """bin/trace_run end to end on this design: pieces of two requests side by side, a request that ends and one that
    takes its pages, both number formats."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = og.make_config(n_layers=3, weights_of={2: 1}, mlps=(True, False, False))
    W = og.make_weights(cfg, seed=17)
    d = str(tmp_path / "m")
    og.save_model_dir(d, cfg, W)
    P = {"a": prompt(cfg, 50, 80), "b": prompt(cfg, 31, 81), "c": prompt(cfg, 40, 82)}
    want = {k: og.forward(cfg, W, v).numpy() for k, v in P.items()}
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": P["a"][:30], "want": [0, 29]}, {"id": "b", "tokens": P["b"][:2], "want": []}], "end": []},
        {"step": 1, "entries": [{"id": "b", "tokens": P["b"][2:], "want": [0, 28]}, {"id": "a", "tokens": P["a"][30:31], "want": [0]}], "end": ["b"]},
        {"step": 2, "entries": [{"id": "a", "tokens": P["a"][31:], "want": [18]}, {"id": "c", "tokens": P["c"], "want": [39, 5]}], "end": ["a", "c"]},
    ]
    rows = {0: [("a", 0), ("a", 29)], 1: [("b", 2), ("b", 30), ("a", 30)], 2: [("a", 49), ("c", 39), ("c", 5)]}
    for dtype in ("float32", "bfloat16"):
        out = str(tmp_path / ("out_" + dtype))
        r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", d, "--dtype", dtype, "--out", out, "--max-tokens", "128"],
                           input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
        for st, rr in rows.items():
            got = np.fromfile(os.path.join(out, f"{st}.f32"), dtype="<f4").reshape(len(rr), cfg["vocab"])
            check(got, np.stack([want[k][i] for k, i in rr]), dtype, f"step {st}")
