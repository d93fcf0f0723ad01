"""Kefurax through libssdk (HybridRunner / LLM) against the plain float64 oracle of tests/kefurax_plain.py, on small
random checkpoints of sizes of their own.  float32 storage is the sharp comparison (a wrong key, tap, edge or state shows
as an error of 1e-2 .. 1, rounding as 1e-6); bfloat16 runs check what the product kernels round."""
import numpy as np
import pytest
import torch

from tests import kefurax_util as U

pytestmark = pytest.mark.gpu

F32_TOL = 3e-4
BF16_TOL = 6e-2


def _load(path, dtype="float32", **kw):
    from ssd_b200.hybrid import HybridRunner, HybridSpec, load_hybrid_weights
    spec = HybridSpec.from_dir(path)
    w = load_hybrid_weights(path, spec, {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype], "cuda:0")
    args = dict(dtype=dtype, max_tokens=512, max_seqs=4, block_size=16, num_blocks=40, n_slots=4, max_model_len=512)
    args.update(kw)
    return HybridRunner(spec, w, **args)


def _runner(tmp_path, cfg, seed=0, dtype="float32", tensors=None, **kw):
    tensors = tensors or U.random_tensors(cfg, seed)
    path = U.write_checkpoint(str(tmp_path / f"ckpt{seed}"), cfg, tensors)
    return _load(path, dtype, **kw), U.PlainModel(cfg, tensors), path


def _tokens(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def _pages(n, block, first=0):
    return list(range(first, first + -(-n // block)))


GQA = U.attention(heads=6, kv_heads=2, dim=10, vdim=7, scale=0.3, dims=6)
FULL = [U.parallel(mlp=U.dense()), U.mamba1(), U.rglru(mlp=U.dense(12)),
        U.parallel(left=GQA, right=U.delta(heads=3, kv_heads=1, dim=9, vdim=12, conv=4), left_scale=1.1, right_scale=0.4),
        U.mamba1(inner=33, state=17, dt_rank=5, conv=2, mlp=U.dense(40)), U.rglru(width=30, blocks=3, conv=2)]

MIXERS = {
    "rglru": U.rglru(),
    "rglru-one-block-five-taps": U.rglru(width=17, blocks=1, conv=5),
    "rglru-one-tap": U.rglru(width=32, blocks=4, conv=1),
    "mamba1": U.mamba1(),
    "mamba1-state-40": U.mamba1(inner=12, state=40, dt_rank=1, conv=4),
    "mamba1-state-70": U.mamba1(inner=9, state=70, dt_rank=4, conv=2),
    "mamba1-state-beyond-registers": U.mamba1(inner=5, state=130, dt_rank=2, conv=3),
    "pair": U.parallel(),
    "pair-attention-only": U.parallel(right_scale=0.0),
    "pair-delta-only": U.parallel(left_scale=0.0),
    "pair-grouped": U.parallel(left=GQA, right=U.delta(heads=6, kv_heads=2, dim=5, vdim=3)),
    "pair-one-kv-head-full-rotation": U.parallel(left=U.attention(heads=5, kv_heads=1, dim=6, vdim=11, dims=6, scaling=None),
                                                 right=U.delta(heads=1, kv_heads=1, dim=40, vdim=33, conv=2)),
    "pair-no-rotation": U.parallel(left=U.attention(heads=2, kv_heads=2, dim=5, vdim=5, dims=0)),
    "pair-wide-delta-head": U.parallel(right=U.delta(heads=2, kv_heads=2, dim=70, vdim=40, conv=5)),
    "pair-delta-head-132": U.parallel(right=U.delta(heads=1, kv_heads=1, dim=132, vdim=8)),
    "pair-delta-head-beyond-registers": U.parallel(right=U.delta(heads=1, kv_heads=1, dim=40, vdim=520, conv=2)),
    "pair-unequal-scaling": U.parallel(left=U.attention(heads=2, kv_heads=1, dim=16, vdim=4, dims=12,
                                                        scaling={"factor": 16.0, "original": 40, "fast": 4.0, "slow": 2.0})),
}


@pytest.mark.parametrize("name", list(MIXERS))
def test_each_mixer_alone(tmp_path, name):
    cfg = U.config([MIXERS[name]])
    r, plain, _ = _runner(tmp_path, cfg)
    toks = _tokens(37, cfg["vocab"], 1)
    lg, _, res = r.forward([(toks, 0, 2, _pages(37, 16, 5), list(range(37)))], residual=True)
    lo = []
    ref = plain.run(toks, layers_out=lo)
    assert U.rel_err(res[0], lo[0].numpy()) < F32_TOL
    assert U.rel_err(lg, ref.numpy()) < F32_TOL
    # the same prompt in two portions and a single token, in another slot and other pages
    out = [r.forward([(toks[a:b], a, 0, _pages(37, 16, 20), list(range(b - a)))])[0] for a, b in ((0, 2), (2, 36), (36, 37))]
    assert U.rel_err(np.concatenate(out), ref.numpy()) < F32_TOL


def test_feed_forward_alone(tmp_path):
    cfg = U.config([U.rglru(mlp=U.dense(28))], mult=1.0)
    tensors = U.random_tensors(cfg, 3)
    tensors["l0.mix.o"].zero_()  # a mixer that returns zero adds nothing: norm(0) = 0
    r, plain, _ = _runner(tmp_path, cfg, tensors=tensors)
    toks = _tokens(90, cfg["vocab"], 4)
    _, _, res = r.forward([(toks, 0, 0, [], list(range(90)))], residual=True)
    lo = []
    plain.run(toks, layers_out=lo)
    assert U.rel_err(res[0], lo[0].numpy()) < F32_TOL
    x0 = tensors["embed"][torch.tensor(toks)].double() * cfg["embedding"]["scale"]
    assert (lo[0] - x0).abs().max() > 0.1  # the feed-forward did move the residual stream


def test_prefill_portions_and_token_by_token(tmp_path):
    cfg = U.config(FULL)
    r, plain, _ = _runner(tmp_path, cfg)
    n = 150
    toks = _tokens(n, cfg["vocab"], 5)
    ref = plain.run(toks).numpy()
    whole, _ = r.forward([(toks, 0, 0, _pages(n, 16), list(range(n)))])
    assert U.rel_err(whole, ref) < F32_TOL
    # portions of several sizes, down to two tokens (shorter than the convolutions), cut inside pages; then single tokens
    for sizes, slot, first in (([2, 3, 16, 5, 2, 31, 2, 17, 64], 1, 10), ([1] * n, 2, 20), ([47, 2, 2, 2, 1, 2], 3, 30)):
        out, pos, k = [], 0, 0
        while pos < n:
            c = min(sizes[k % len(sizes)], n - pos)
            lg, _ = r.forward([(toks[pos:pos + c], pos, slot, _pages(n, 16, first), list(range(c)))])
            out.append(lg)
            pos, k = pos + c, k + 1
        got = np.concatenate(out)
        assert U.rel_err(got, ref) < F32_TOL
        assert np.abs(got - whole).max() < 1e-4 * np.abs(whole).max()


def test_batch_of_unequal_requests_equals_each_alone(tmp_path):
    cfg = U.config(FULL)
    r, plain, _ = _runner(tmp_path, cfg)
    lens = [70, 9, 33, 1]
    seqs = [_tokens(n, cfg["vocab"], 10 + i) for i, n in enumerate(lens)]
    alone = [r.forward([(s, 0, 0, _pages(len(s), 16), list(range(len(s))))])[0] for s in seqs]
    # step 1: portions of requests 0, 1 and 2 + the whole of request 3; step 2: the rests, one of them a single token
    cut = [40, 8, 20, 1]
    pages = [_pages(n, 16, 8 * i) for i, n in enumerate(lens)]
    a, _ = r.forward([(seqs[i][:cut[i]], 0, i, pages[i], list(range(cut[i]))) for i in range(4)])
    b, _ = r.forward([(seqs[i][cut[i]:], cut[i], i, pages[i], list(range(lens[i] - cut[i]))) for i in (2, 1, 0)])
    got = {0: [], 1: [], 2: [], 3: []}
    o = 0
    for i in range(4):
        got[i].append(a[o:o + cut[i]]); o += cut[i]
    o = 0
    for i in (2, 1, 0):
        got[i].append(b[o:o + lens[i] - cut[i]]); o += lens[i] - cut[i]
    for i in range(4):
        g = np.concatenate(got[i])
        assert np.abs(g - alone[i]).max() < 2e-5 * np.abs(alone[i]).max(), f"request {i} depends on its batch"
        assert U.rel_err(g, plain.run(seqs[i]).numpy()) < F32_TOL


def test_pages_and_slots_are_reused(tmp_path, monkeypatch):
    """Requests come and go through the engine's managers: a later request gets the pages and the state slot that an
    earlier one dirtied (recurrent matrices, convolution histories, keys and values), in another order."""
    from ssd_b200.engine.block_manager import BlockManager
    from ssd_b200.engine.sequence import Sequence
    from ssd_b200.engine.state_manager import StateSlotManager
    cfg = U.config(FULL)
    r, plain, _ = _runner(tmp_path, cfg, num_blocks=8, n_slots=2)
    monkeypatch.setattr(Sequence, "block_size", 16)
    bm, sm = BlockManager(8, 16, prefix_reuse=False), StateSlotManager(2)
    prompts = [_tokens(n, cfg["vocab"], 20 + i) for i, n in enumerate([50, 40, 45, 30, 3])]
    used_pages, used_slots, live = [], [], []
    for k, toks in enumerate(prompts):
        if len(live) == 2:  # the pools are full: the older request ends
            old = live.pop(0)
            bm.deallocate(old); sm.free(old)
        s = Sequence(toks)
        bm.allocate(s); sm.allocate(s)
        live.append(s)
        used_pages.append(tuple(s.block_table)); used_slots.append(s.state_slot)
        half = len(toks) // 2
        a, _ = r.forward([(toks[:half], 0, s.state_slot, s.block_table, list(range(half)))])
        b, _ = r.forward([(toks[half:], half, s.state_slot, s.block_table, list(range(len(toks) - half)))])
        assert U.rel_err(np.concatenate([a, b]), plain.run(toks).numpy()) < F32_TOL, f"request {k}"
    assert len(set(used_slots)) < len(used_slots) and len({p for t in used_pages for p in t}) <= 8


def test_far_keys_page_borders_and_sink(tmp_path):
    """Attention made sharp: unit-RMS queries and keys with a large score scale put nearly all weight on ONE key, wherever
    it lies (hundreds of tokens back, on either side of a page border), in prompts and in decoding; where every score is
    negative the constant in the denominator takes most of the weight."""
    left = U.attention(heads=4, kv_heads=2, dim=8, vdim=8, scale=2.5, dims=8, base=50.0)
    cfg = U.config([U.parallel(left=left, left_scale=1.5, right_scale=0.1, mlp=U.dense()),
                    U.parallel(left=U.attention(heads=2, kv_heads=1, dim=6, vdim=6, scale=1.5, dims=2), right_scale=0.2)])
    tensors = U.random_tensors(cfg, 7)
    r, plain, _ = _runner(tmp_path, cfg, tensors=tensors, max_model_len=384, num_blocks=24, n_slots=1)
    n, tail = 330, 70
    toks = _tokens(n, cfg["vocab"], 8)
    ref = plain.run(toks).numpy()
    pages = list(range(23, 23 - 21, -1))
    out = [r.forward([(toks[:n - tail], 0, 0, pages, list(range(n - tail)))])[0]]
    for p in range(n - tail, n):  # decoding walks over four page borders
        out.append(r.forward([([toks[p]], p, 0, pages, [0])])[0])
    got = np.concatenate(out)
    per_pos = np.sqrt(((got - ref) ** 2).mean(-1)) / np.sqrt((ref ** 2).mean())
    assert per_pos.max() < 2e-3, f"worst position {int(per_pos.argmax())}"
    # the comparison does rest on far keys: another token at position 3 moves the logits hundreds of positions later
    toks2 = list(toks)
    toks2[3] = (toks[3] + 1) % cfg["vocab"]
    ref2 = plain.run(toks2).numpy()
    moved = np.sqrt(((ref2 - ref) ** 2).mean(-1))[200:] / np.sqrt((ref ** 2).mean())
    assert moved.max() > 20 * 2e-3
    got2, _ = r.forward([(toks2, 0, 0, pages, list(range(n)))])
    assert U.rel_err(got2, ref2) < 2e-3
    # and on the sink: a softmax without the 1 in its denominator gives visibly other logits
    import functools
    from tests import kefurax_plain as P
    keep = P.sink_attention
    P.sink_attention = functools.partial(keep, sink=0.0)
    try:
        plain_softmax = plain.run(toks[:40]).numpy()
    finally:
        P.sink_attention = keep
    assert U.rel_err(plain_softmax, ref[:40]) > 0.02


def test_decoding_sequences_of_unequal_context_share_a_step(tmp_path):
    """Three sequences decode together at contexts of a few, ~150 and ~300 tokens beside a prompt portion of a fourth: the
    single-token rows take the split-context attention (some splits of the short sequence hold no key at all), the
    portion the GEMM path, in one call."""
    cfg = U.config([U.parallel(left=U.attention(heads=6, kv_heads=3, dim=8, vdim=10, scale=1.5, dims=8), mlp=U.dense()),
                    U.rglru(), U.mamba1(), U.parallel(left=U.attention(heads=5, kv_heads=5, dim=6, vdim=40, scale=1.0, dims=4))])
    r, plain, _ = _runner(tmp_path, cfg, seed=5, max_tokens=512, max_model_len=512, num_blocks=64)
    lens, steps = [3, 150, 300, 90], 6
    seqs = [_tokens(n + steps, cfg["vocab"], 90 + i) for i, n in enumerate(lens)]
    refs = [plain.run(s).numpy() for s in seqs]
    pages = [_pages(len(s), 16, first) for s, first in zip(seqs, (58, 40, 5, 30))]
    for i in range(3):  # prompts of the decoding sequences, each alone
        r.forward([(seqs[i][:lens[i]], 0, i, pages[i], [lens[i] - 1])])
    got = [[] for _ in seqs]
    for t in range(steps):
        ents = [([seqs[i][lens[i] + t]], lens[i] + t, i, pages[i], [0]) for i in range(3)]
        lo, hi = 16 * t, (16 * (t + 1) if t < steps - 1 else len(seqs[3]))
        ents.insert(1, (seqs[3][lo:hi], lo, 3, pages[3], list(range(hi - lo))))
        lg, _ = r.forward(ents)
        got[0].append(lg[0:1]); got[3].append(lg[1:1 + hi - lo]); got[1].append(lg[1 + hi - lo:2 + hi - lo]); got[2].append(lg[2 + hi - lo:])
    for i in range(3):
        assert U.rel_err(np.concatenate(got[i]), refs[i][lens[i]:]) < 2e-3, f"decoding sequence {i}"
    assert U.rel_err(np.concatenate(got[3]), refs[3]) < 2e-3


def test_first_tokens_and_long_decoding(tmp_path):
    cfg = U.config(FULL)
    r, plain, _ = _runner(tmp_path, cfg, seed=2)
    for n in (1, 2, 3):
        toks = _tokens(n, cfg["vocab"], 30 + n)
        lg, _ = r.forward([(toks, 0, 1, [4], list(range(n)))])
        assert U.rel_err(lg, plain.run(toks).numpy()) < F32_TOL
    toks = _tokens(260, cfg["vocab"], 40)
    ref = plain.run(toks).numpy()
    out = [r.forward([(toks[:4], 0, 0, _pages(260, 16), [0, 1, 2, 3])])[0]]
    for p in range(4, 260):
        out.append(r.forward([([toks[p]], p, 0, _pages(260, 16), [0])])[0])
    got = np.concatenate(out)
    per_pos = np.sqrt(((got - ref) ** 2).mean(-1)) / np.sqrt((ref ** 2).mean())
    assert per_pos.max() < 5 * F32_TOL, f"worst position {int(per_pos.argmax())}"


def test_long_batches_are_split_into_calls(tmp_path):
    cfg = U.config(FULL[:4])
    r, plain, _ = _runner(tmp_path, cfg, max_tokens=48, max_seqs=2, max_logit_rows=48)
    seqs = [_tokens(n, cfg["vocab"], 50 + i) for i, n in enumerate([100, 7, 30])]
    lg, _ = r.forward([(s, 0, i, _pages(len(s), 16, 8 * i), [0, len(s) - 1]) for i, s in enumerate(seqs)])
    for i, s in enumerate(seqs):
        ref = plain.run(s).numpy()
        assert U.rel_err(lg[2 * i:2 * i + 2], ref[[0, len(s) - 1]]) < F32_TOL


@pytest.mark.parametrize("width", [40, 128, 36], ids=["rows-16B-aligned", "tcgen05-shapes", "unaligned"])
def test_bfloat16_storage(tmp_path, width):
    """bf16 weights / activations / cache with fp32 accumulation, residual, state, gates and scores.  The width picks the
    product kernel: 128 puts the dense projections on the tcgen05 GEMM, 40 on the mma.sync tile, 36 on the FMA tile."""
    big = [U.parallel(left=U.attention(heads=4, kv_heads=2, dim=32, vdim=32, scale=0.2, dims=16), right=U.delta(heads=2, kv_heads=1, dim=32, vdim=64, conv=4),
                      mlp=U.dense(64)), U.rglru(width=64, blocks=2), U.mamba1(inner=64, state=16, dt_rank=8, mlp=U.dense(64))]
    cfg = U.config(FULL[:3] + big, width=width)
    r, plain, _ = _runner(tmp_path, cfg, dtype="bfloat16")
    n = 120
    toks = _tokens(n, cfg["vocab"], 60)
    ref = plain.run(toks).numpy()
    whole, _ = r.forward([(toks, 0, 0, _pages(n, 16), list(range(n)))])
    assert U.rel_err(whole, ref) < BF16_TOL
    out, pos = [], 0
    for c in [2, 30, 3, 64, 2] + [1] * 19:
        out.append(r.forward([(toks[pos:pos + c], pos, 1, _pages(n, 16, 9), list(range(c)))])[0])
        pos += c
    assert U.rel_err(np.concatenate(out), whole) < 2e-2


def test_bfloat16_calls_of_many_rows(tmp_path):
    """More rows than one tile of the tcgen05 GEMM holds (256): two prompts of unequal length in one call, against the
    oracle and against portions that each fit a single tile."""
    cfg = U.config([U.parallel(left=U.attention(heads=4, kv_heads=2, dim=32, vdim=32, scale=0.2, dims=16),
                               right=U.delta(heads=2, kv_heads=2, dim=32, vdim=32, conv=4), mlp=U.dense(64)),
                    U.mamba1(inner=128, state=8, dt_rank=8), U.rglru(width=64, blocks=2, mlp=U.dense(128))], width=128, vocab=96)
    r, plain, _ = _runner(tmp_path, cfg, dtype="bfloat16", max_tokens=1024, max_model_len=512, num_blocks=64)
    seqs = [_tokens(330, cfg["vocab"], 80), _tokens(271, cfg["vocab"], 81)]
    refs = [plain.run(s).numpy() for s in seqs]
    lg, _ = r.forward([(s, 0, i, _pages(len(s), 16, 30 * i), list(range(len(s)))) for i, s in enumerate(seqs)])
    got = [lg[:330], lg[330:]]
    for g, ref in zip(got, refs):
        assert U.rel_err(g, ref) < BF16_TOL
    out, pos = [], 0
    for c in [200, 100, 30]:
        out.append(r.forward([(seqs[0][pos:pos + c], pos, 2, _pages(330, 16, 30), list(range(c)))])[0])
        pos += c
    assert U.rel_err(np.concatenate(out), got[0]) < 2e-2


def test_greedy_generation_through_llm(tmp_path):
    """The public entry point: LLM.generate with the engine's scheduler (three prompts, two state slots: the third
    waits for a slot and gets a used one), temperature 0, against the oracle's greedy continuation."""
    from ssd_b200 import LLM, SamplingParams
    cfg = U.config(FULL[:4], vocab=64)
    tensors = U.random_tensors(cfg, 11)
    path = U.write_checkpoint(str(tmp_path / "gen"), cfg, tensors)
    plain = U.PlainModel(cfg, tensors)
    prompts = [_tokens(n, cfg["vocab"], 70 + i) for i, n in enumerate([21, 5, 40])]
    llm = LLM(path, dtype="float32", kvcache_block_size=16, max_model_len=128, max_num_batched_tokens=128, max_num_seqs=2)
    try:
        outs, _ = llm.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=12, ignore_eos=True), use_tqdm=False)
    finally:
        llm.exit()
    for p, o in zip(prompts, outs):
        assert o["token_ids"] == plain.greedy(p, 12)
