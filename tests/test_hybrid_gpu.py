"""Layer-list models (the Safupel design) in the engine against the plain float64 oracle (oracle/hybrid.py): every
mechanism alone, whole prompts against pieces and token-by-token decoding, mixed batches, reused pages and state slots,
chunk edges and far keys with peaked scores, the first tokens, long decoding, odd sizes, and greedy generation through
the scheduler.  float32 engines give the sharp comparison; bfloat16 ones are held to a rounding-sized bound."""
import numpy as np
import pytest
import torch

from oracle import hybrid as oh

pytestmark = pytest.mark.gpu

FULL = dict(layers=("parallel", "rglru", "parallel", "rglru"), mlps=("moe", "dense", "dense", "moe-noshared"))


def make_engine(kge, tmp_path, cfg, W, dtype="float32", tokens=512, bs=16, seqs=4, name="m", batched=0):
    d = str(tmp_path / name)
    oh.save_model_dir(d, cfg, W)
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


def check(got, want, dtype, what=""):
    want = want.numpy() if isinstance(want, torch.Tensor) else want
    scale = np.sqrt((want ** 2).mean())
    err = np.sqrt(((got - want) ** 2).mean(-1)) / scale
    lim = 2e-4 if dtype == "float32" else 4e-2
    assert err.max() < lim, f"{what}: worst row {err.argmax()} is {err.max():.3g} of the logits' size (limit {lim})"


def prompt(cfg, n, seed=1):
    return torch.randint(0, cfg["vocab"], (n,), generator=torch.Generator().manual_seed(seed)).tolist()


ALONE = {
    "rglru": dict(layers=("rglru",), mlps=(None,)),
    "attention": dict(layers=("parallel",), mlps=(None,), right_scale=0.0, chunk=16),
    "mlstm": dict(layers=("parallel",), mlps=(None,), left_scale=0.0),
    "moe": dict(layers=("parallel",), mlps=("moe",), left_scale=0.0, right_scale=0.0),
    "moe-noshared": dict(layers=("parallel",), mlps=("moe-noshared",), left_scale=0.0, right_scale=0.0, top=3),
    "dense": dict(layers=("parallel",), mlps=("dense",), left_scale=0.0, right_scale=0.0),
}


@pytest.mark.parametrize("mech", sorted(ALONE))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mechanism_alone(kge, tmp_path, mech, dtype):
    cfg = oh.make_config(**ALONE[mech])
    W = oh.make_weights(cfg, seed=3)
    toks = prompt(cfg, 45)
    llm = make_engine(kge, tmp_path, cfg, W, dtype)
    got = run_pieces(llm, 0, toks, [45])
    llm.close()
    check(got, oh.forward(cfg, W, toks), dtype, mech)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_decode_and_pieces_agree_with_the_oracle(kge, tmp_path, dtype):
    cfg = oh.make_config(**FULL, chunk=24)
    W = oh.make_weights(cfg, seed=5)
    toks = prompt(cfg, 75)
    want = oh.forward(cfg, W, toks)
    llm = make_engine(kge, tmp_path, cfg, W, dtype)
    for rid, pieces in enumerate([[75], [30] + [1] * 45, [1] * 75, [2, 3, 17, 2, 31, 5, 2, 2, 9, 2], [23, 2, 24, 26], [47, 2, 1, 1, 24]]):
        got = run_pieces(llm, rid, toks, pieces)
        llm.trace_end(rid)
        check(got, want, dtype, f"pieces {pieces[:6]}")
    llm.close()


def test_layer_outputs_match(kge, tmp_path):
    cfg = oh.make_config(**FULL)
    W = oh.make_weights(cfg, seed=6)
    toks = prompt(cfg, 33)
    _, layers = oh.forward(cfg, W, toks, return_layers=True)
    llm = make_engine(kge, tmp_path, cfg, W, "float32")
    buf = np.zeros((4, 33, cfg["width"]), dtype=np.float32)
    llm.set_layer_dump(buf)
    run_pieces(llm, 0, toks, [33])
    llm.set_layer_dump(None)
    llm.close()
    for i, x in enumerate(layers):
        assert np.abs(buf[i] - x.numpy()).max() < 2e-4 * float(x.abs().max()), f"layer {i}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_of_unequal_requests(kge, tmp_path, dtype):
    cfg = oh.make_config(**FULL, chunk=20)
    W = oh.make_weights(cfg, seed=7)
    P = {0: prompt(cfg, 61, 10), 1: prompt(cfg, 9, 11), 2: prompt(cfg, 40, 12), 3: prompt(cfg, 1, 13)}
    want = {r: oh.forward(cfg, W, t).numpy() for r, t in P.items()}
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
        check(np.concatenate(got[r]), want[r], dtype, f"request {r}")


def test_pages_and_slots_are_used_again(kge, tmp_path):
    """Two slots and a pool of 96 tokens: five requests pass through, each starting in a slot and in pages that an
    earlier request filled; each must come out as if it had run alone."""
    cfg = oh.make_config(**FULL, chunk=24)
    W = oh.make_weights(cfg, seed=8)
    llm = make_engine(kge, tmp_path, cfg, W, "float32", tokens=96, bs=16, seqs=2)
    P = {r: prompt(cfg, n, 20 + r) for r, n in enumerate([40, 33, 47, 18, 30])}
    want = {r: oh.forward(cfg, W, t).numpy() for r, t in P.items()}
    got = {}
    got[0] = run_pieces(llm, 0, P[0], [40])
    llm.trace_add(1, P[1][:20])
    a = llm.trace_step([(1, 20, list(range(20)))])
    with pytest.raises(kge.KgeError):                     # no third slot
        llm.trace_add(2, P[2])
        llm.trace_step([(2, 5, [])])
    llm.trace_end(2)
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


@pytest.mark.parametrize("dims", [(12, 20), (32, 40)])       # the per-row kernel; the tensor-core kernel (bfloat16, key size a multiple of 16)
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_chunk_edges_with_peaked_scores(kge, tmp_path, dtype, dims):
    """Attention alone, scores large enough that single keys carry most of the weight: a key that is wrongly seen or
    missed at a chunk's edge, or a page border that is misread, moves the logits far beyond rounding."""
    cfg = oh.make_config(layers=("parallel",), mlps=(None,), right_scale=0.0, chunk=21, scale=1.6 * (12 / dims[0]) ** 0.5, heads=4, kv_heads=1,
                         dim=dims[0], vdim=dims[1])
    W = oh.make_weights(cfg, seed=9)
    toks = prompt(cfg, 70, 30)
    want = oh.forward(cfg, W, toks)
    ref = want.numpy()
    assert np.abs(ref[21] - oh.forward(dict(cfg, layers=[dict(cfg["layers"][0], mixer=dict(cfg["layers"][0]["mixer"], left=dict(
        cfg["layers"][0]["mixer"]["left"], mask={"size": 22})))]), W, toks).numpy()[21]).max() > 0.05      # the edge matters in this setup
    llm = make_engine(kge, tmp_path, cfg, W, dtype, bs=16)
    check(run_pieces(llm, 0, toks, [70]), want, dtype, "whole")
    check(run_pieces(llm, 1, toks, [19] + [1] * 30 + [21]), want, dtype, "decoding over two edges")
    check(run_pieces(llm, 2, toks, [20, 2, 20, 2, 26]), want, dtype, "pieces that straddle the edges")
    llm.close()


def test_far_keys_tensor_core_kernel(kge, tmp_path):
    """bfloat16, 32-wide keys and 56-wide values, several key tiles per warp and a chunk edge in the middle of the prompt;
    grouped heads."""
    cfg = oh.make_config(layers=("parallel",), mlps=(None,), right_scale=0.0, chunk=200, scale=0.7, heads=6, kv_heads=2, dim=32, vdim=56)
    W = oh.make_weights(cfg, seed=15)
    toks = prompt(cfg, 290, 32)
    want = oh.forward(cfg, W, toks)
    llm = make_engine(kge, tmp_path, cfg, W, "bfloat16", bs=64)
    got = np.concatenate([run_pieces(llm, 0, toks[:150], [150]), run_pieces(llm, 0, toks[150:260], [3, 45, 2, 60]), run_pieces(llm, 0, toks[260:], [1] * 30)])
    llm.close()
    check(got, want, "bfloat16")


def test_far_keys_among_hundreds(kge, tmp_path):
    """One long chunk: the second head's distance penalty is weak, so keys hundreds of positions back keep real weight."""
    cfg = oh.make_config(layers=("parallel",), mlps=(None,), right_scale=0.0, chunk=400, scale=1.2, heads=2, kv_heads=2, dim=8, vdim=8)
    W = oh.make_weights(cfg, seed=10)
    toks = prompt(cfg, 330, 31)
    want = oh.forward(cfg, W, toks)
    llm = make_engine(kge, tmp_path, cfg, W, "float32", bs=64)
    got = np.concatenate([run_pieces(llm, 0, toks[:300], [300]), run_pieces(llm, 0, toks[300:], [1] * 30)])
    llm.close()
    check(got, want, "float32")


def test_experts_with_many_routed_rows(kge, tmp_path):
    """A prompt long enough that the routed rows are made contiguous per expert and run as one tensor-core GEMM pair per
    expert (bfloat16; expert width a multiple of 64); the same prompt fed in short pieces takes the grouped kernel."""
    cfg = oh.make_config(layers=("rglru",), mlps=("moe",), experts=6, top=2, expert_ff=64, shared_ff=64, r_width=64, r_blocks=2)
    W = oh.make_weights(cfg, seed=16)
    toks = prompt(cfg, 300, 33)
    want = oh.forward(cfg, W, toks)
    llm = make_engine(kge, tmp_path, cfg, W, "bfloat16", bs=64)
    check(run_pieces(llm, 0, toks, [300]), want, "bfloat16", "one step")
    llm.trace_end(0)
    check(run_pieces(llm, 1, toks, [280, 7, 13]), want, "bfloat16", "pieces")
    llm.close()


def test_first_tokens(kge, tmp_path):
    cfg = oh.make_config(**FULL)
    W = oh.make_weights(cfg, seed=11)
    llm = make_engine(kge, tmp_path, cfg, W, "float32")
    for rid, n in enumerate([1, 2, 3, 5]):
        toks = prompt(cfg, n, 40 + n)
        got = run_pieces(llm, rid, toks, [n])
        llm.trace_end(rid)
        check(got, oh.forward(cfg, W, toks), "float32", f"{n} tokens")
    llm.close()


def test_long_decoding(kge, tmp_path):
    cfg = oh.make_config(**FULL, chunk=32)
    W = oh.make_weights(cfg, seed=12)
    toks = prompt(cfg, 200, 50)
    llm = make_engine(kge, tmp_path, cfg, W, "float32")
    got = run_pieces(llm, 0, toks, [4] + [1] * 196)
    llm.close()
    check(got, oh.forward(cfg, W, toks), "float32")


@pytest.mark.parametrize("sizes", [
    dict(heads=3, kv_heads=3, dim=16, vdim=16, m_heads=1, m_dim=16, m_vdim=16, r_blocks=1, r_conv=1, experts=2, top=1, chunk=7),
    dict(vocab=53, width=40, heads=6, kv_heads=2, dim=10, vdim=14, m_heads=2, m_dim=6, m_vdim=36, r_width=60, r_blocks=5, r_conv=7,
         ff=50, experts=9, top=4, expert_ff=11, shared_ff=13, chunk=64, left_scale=0.7, right_scale=1.3, gate_cap=4.0, logit_scale=2.0, eps=1e-3),
])
def test_other_sizes(kge, tmp_path, sizes):
    cfg = oh.make_config(**FULL, **sizes)
    W = oh.make_weights(cfg, seed=13)
    toks = prompt(cfg, 50, 60)
    want = oh.forward(cfg, W, toks)
    llm = make_engine(kge, tmp_path, cfg, W, "float32")
    check(run_pieces(llm, 0, toks, [50]), want, "float32", "whole")
    check(run_pieces(llm, 1, toks, [13, 2, 1, 1, 1, 32]), want, "float32", "pieces")
    llm.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_scheduler(kge, tmp_path, dtype):
    """LLM.generate: the continuous-batching scheduler cuts the prompts into 16-token steps, admits the third request
    when a slot frees up, and samples greedily."""
    cfg = oh.make_config(**FULL, chunk=24)
    W = oh.make_weights(cfg, seed=14)
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
            lg = oh.forward(cfg, W, toks)[-1]
            best = int(torch.argmax(lg))
            if g != best:
                gap = float(lg[best] - lg[g])
                assert gap < (1e-3 if dtype == "float32" else 0.15), f"token {k}: chose {g}, oracle {best} leads by {gap}"
            toks.append(g)


def test_trace_runner_command_line(kge, tmp_path):
    """bin/trace_run end to end: JSON steps on stdin (pieces of two requests side by side, a request that ends and one
    that takes its slot and pages), float32 files out, 'done <step>' lines; and exit code 3 for a family without float32."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = oh.make_config(layers=("rglru", "parallel", "parallel"), mlps=("dense", "moe", None), chunk=24)
    W = oh.make_weights(cfg, seed=17)
    d = str(tmp_path / "m")
    oh.save_model_dir(d, cfg, W)
    P = {"a": prompt(cfg, 50, 80), "b": prompt(cfg, 31, 81), "c": prompt(cfg, 40, 82)}
    want = {k: oh.forward(cfg, W, v).numpy() for k, v in P.items()}
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
    from oracle import model as om
    lcfg = om.CONFIGS["tiny-llama"]
    ld = str(tmp_path / "llama")
    om.save_model_dir(ld, lcfg, om.make_weights(lcfg, seed=0))
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", ld, "--dtype", "float32", "--out", str(tmp_path / "o2"),
                        "--max-tokens", "128"], input="", capture_output=True, text=True, timeout=600)
    assert r.returncode == 3, (r.returncode, r.stderr[-500:])

