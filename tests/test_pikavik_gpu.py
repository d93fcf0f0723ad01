"""Pikavik through libssdk (HybridRunner / LLM) against the plain float64 oracle of tests/pikavik_plain.py, on small
random checkpoints of sizes of their own.  float32 storage is the sharp comparison (a wrong key, edge or state shows as
an error of 1e-2 .. 1, rounding as 1e-6); bfloat16 runs are compared where no discrete choice (expert routing) can flip."""
import numpy as np
import pytest
import torch

from tests import pikavik_util as U
from tests.pikavik_plain import PlainModel

pytestmark = pytest.mark.gpu

F32_TOL = 3e-4
BF16_TOL = 6e-2


def _runner(tmp_path, cfg, seed=0, dtype="float32", **kw):
    from ssd_b200.hybrid import HybridRunner, HybridSpec, load_hybrid_weights
    tensors = U.random_tensors(cfg, seed)
    path = U.write_checkpoint(str(tmp_path / f"ckpt{seed}"), cfg, tensors)
    spec = HybridSpec.from_dir(path)
    w = load_hybrid_weights(path, spec, {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype], "cuda:0")
    args = dict(dtype=dtype, max_tokens=512, max_seqs=4, block_size=16, num_blocks=40, n_slots=4, max_model_len=512)
    args.update(kw)
    return HybridRunner(spec, w, **args), PlainModel(cfg, tensors), path


def _tokens(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def _pages(n, block, first=0):
    return list(range(first, first + -(-n // block)))


FULL = [U.mlstm(mlp=U.moe()), U.wkv(mlp=U.moe(experts=4, top=1, groups=1, keep=1, shared_ff=0)),
        U.latent(mlp=U.moe(experts=6, top=2, groups=6, keep=3, ff=12, shared_ff=20, limit=0.7)),
        U.wkv(heads=1, dim=24, rank=3), U.mlstm(heads=3, dim=6, vdim=11, cap=4.0, mlp=U.moe(scale=1.0)),
        U.latent(heads=1, dim=6, rot_dim=4, vdim=5, kv_rank=9, q_rank=7, scale=0.5, base=100.0)]


@pytest.mark.parametrize("layer", [U.wkv(), U.wkv(heads=3, dim=20, rank=2), U.mlstm(), U.mlstm(heads=1, dim=33, vdim=7, cap=3.0),
                                   U.latent(), U.latent(heads=5, dim=4, rot_dim=12, vdim=3, kv_rank=7, q_rank=30, scale=1.0),
                                   U.latent(rot_dim=10, dims=6)],
                         ids=["wkv", "wkv-wide", "mlstm", "mlstm-one-head", "latent", "latent-odd", "latent-part-rot"])
def test_each_mixer_alone(tmp_path, layer):
    cfg = U.config([layer])
    r, plain, _ = _runner(tmp_path, cfg)
    toks = _tokens(37, cfg["vocab"], 1)
    lg, _, res = r.forward([(toks, 0, 2, _pages(37, 16, 5), list(range(37)))], residual=True)
    lo = []
    ref = plain.run(toks, layers_out=lo)
    assert U.rel_err(res[0], lo[0].numpy()) < F32_TOL
    assert U.rel_err(lg, ref.numpy()) < F32_TOL


@pytest.mark.parametrize("mlp", [U.moe(), U.moe(experts=4, top=1, groups=1, keep=1, shared_ff=0),
                                 U.moe(experts=6, top=2, groups=6, keep=3, ff=12, shared_ff=20, limit=0.7),
                                 U.moe(experts=8, top=4, groups=2, keep=2, scale=1.0, shared_ff=5)],
                         ids=["grouped", "top1-no-shared", "one-expert-groups", "all-groups"])
def test_feed_forward_alone(tmp_path, mlp):
    cfg = U.config([U.mlstm(mlp=mlp)])
    tensors = U.random_tensors(cfg, 3)
    tensors["l0.ls1"].zero_()  # the mixer branch is switched off by its layer scale
    path = U.write_checkpoint(str(tmp_path / "ff"), cfg, tensors)
    from ssd_b200.hybrid import HybridRunner, HybridSpec, load_hybrid_weights
    spec = HybridSpec.from_dir(path)
    r = HybridRunner(spec, load_hybrid_weights(path, spec, torch.float32, "cuda:0"), dtype="float32", max_tokens=256,
                     block_size=16, num_blocks=8, n_slots=2, max_model_len=128)
    toks = _tokens(90, cfg["vocab"], 4)
    _, _, res = r.forward([(toks, 0, 0, [], list(range(90)))], residual=True)
    lo = []
    PlainModel(cfg, tensors).run(toks, layers_out=lo)
    assert U.rel_err(res[0], lo[0].numpy()) < F32_TOL


def test_prefill_portions_and_token_by_token(tmp_path):
    cfg = U.config(FULL)
    r, plain, _ = _runner(tmp_path, cfg)
    n = 150
    toks = _tokens(n, cfg["vocab"], 5)
    ref = plain.run(toks).numpy()
    whole, _ = r.forward([(toks, 0, 0, _pages(n, 16), list(range(n)))])
    assert U.rel_err(whole, ref) < F32_TOL
    # portions of several sizes, down to two tokens, cut inside pages; then single tokens
    for sizes, slot, first in (([2, 3, 16, 5, 2, 31, 2, 17, 64], 1, 10), ([1] * n, 2, 20), ([47, 2, 2, 2], 3, 30)):
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
        assert np.abs(g - alone[i]).max() < 1e-5 * np.abs(alone[i]).max(), f"request {i} depends on its batch"
        assert U.rel_err(g, plain.run(seqs[i]).numpy()) < F32_TOL


def test_pages_and_slots_are_reused(tmp_path, monkeypatch):
    """Requests come and go through the engine's Scheduler: a later request gets the pages and the state slot that an
    earlier one dirtied, in another order."""
    from ssd_b200.engine.block_manager import BlockManager
    from ssd_b200.engine.sequence import Sequence
    from ssd_b200.engine.state_manager import StateSlotManager
    cfg = U.config(FULL)
    r, plain, _ = _runner(tmp_path, cfg, num_blocks=8, n_slots=2)
    monkeypatch.setattr(Sequence, "block_size", 16)
    bm, sm = BlockManager(8, 16, prefix_reuse=False), StateSlotManager(2)
    prompts = [_tokens(n, cfg["vocab"], 20 + i) for i, n in enumerate([50, 40, 45, 30])]
    used_pages, used_slots = [], []
    live = []
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
    """Latent attention made sharp: a large score scale puts nearly all weight on ONE key, wherever it lies (hundreds of
    tokens back, on either side of a page border), and sinks of +-4 take or leave a visible share of the denominator."""
    layer = U.latent(heads=4, dim=8, rot_dim=8, vdim=8, kv_rank=12, q_rank=12, scale=6.0)
    cfg = U.config([layer, U.latent(heads=2, dim=6, rot_dim=4, vdim=6, kv_rank=8, q_rank=8, scale=3.0, mlp=U.moe())])
    tensors = U.random_tensors(cfg, 7)
    tensors["l0.mix.sink"] = torch.tensor([4.0, -4.0, 1.0, 0.0])
    tensors["l1.mix.sink"] = torch.tensor([-2.0, 3.0])
    path = U.write_checkpoint(str(tmp_path / "sharp"), cfg, tensors)
    from ssd_b200.hybrid import HybridRunner, HybridSpec, load_hybrid_weights
    spec = HybridSpec.from_dir(path)
    r = HybridRunner(spec, load_hybrid_weights(path, spec, torch.float32, "cuda:0"), dtype="float32", max_tokens=512,
                     block_size=16, num_blocks=24, n_slots=1, max_model_len=384)
    plain = PlainModel(cfg, tensors)
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
    assert moved.max() > 50 * 2e-3
    got2, _ = r.forward([(toks2, 0, 0, pages, list(range(n)))])
    assert U.rel_err(got2, ref2) < 2e-3
    # and on the sink: without it the first head's output would be ~50 times larger at short contexts
    t0 = dict(tensors)
    t0["l0.mix.sink"] = torch.tensor([-30.0, -30.0, -30.0, -30.0])
    assert U.rel_err(PlainModel(cfg, t0).run(toks[:40]).numpy(), ref[:40]) > 0.05


def test_decoding_sequences_of_unequal_context_share_a_step(tmp_path):
    """Three sequences decode together at contexts of a few, ~150 and ~300 tokens beside a prompt portion of a fourth: the
    single-token rows take the split-context attention (some splits of the short sequence hold no key at all), the
    portion the GEMM path, in one call.  Sharp scores (large scale) make a wrong or missing far key visible."""
    cfg = U.config([U.latent(heads=3, dim=8, rot_dim=8, vdim=10, kv_rank=12, q_rank=12, scale=4.0, mlp=U.moe()),
                    U.wkv(), U.latent(heads=5, dim=6, rot_dim=4, vdim=6, kv_rank=9, q_rank=8, scale=2.0)])
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
    cfg = U.config(FULL[:3])
    r, plain, _ = _runner(tmp_path, cfg, max_tokens=48, max_seqs=2, max_logit_rows=48)
    seqs = [_tokens(n, cfg["vocab"], 50 + i) for i, n in enumerate([100, 7, 30])]
    lg, _ = r.forward([(s, 0, i, _pages(len(s), 16, 8 * i), [0, len(s) - 1]) for i, s in enumerate(seqs)])
    for i, s in enumerate(seqs):
        ref = plain.run(s).numpy()
        assert U.rel_err(lg[2 * i:2 * i + 2], ref[[0, len(s) - 1]]) < F32_TOL


@pytest.mark.parametrize("width", [40, 128, 36], ids=["rows-16B-aligned", "tcgen05-shapes", "unaligned"])
def test_bfloat16_storage(tmp_path, width):
    """bf16 weights / activations / cache with fp32 accumulation, residual, state and scores.  Every expert is chosen
    (top == experts), so no routing decision can flip between the oracle and the rounded run.  The width picks the
    product kernel: 128 puts the dense projections on the tcgen05 GEMM, 40 on the mma.sync tile, 36 on the FMA tile."""
    every = dict(experts=4, top=4, groups=2, keep=2)
    cfg = U.config([U.mlstm(mlp=U.moe(**every)), U.wkv(mlp=U.moe(**every)), U.latent(mlp=U.moe(**every)), U.wkv(),
                    U.mlstm(heads=3, dim=6, vdim=11), U.wkv(heads=2, dim=32, rank=64), U.latent(heads=2, dim=32, rot_dim=16, vdim=32, kv_rank=64, q_rank=64)],
                   width=width)
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
    # single-token rows take the fused decode attention, which keeps its weights in fp32: equal up to bf16 rounding
    assert U.rel_err(np.concatenate(out), whole) < 1e-2


def test_bfloat16_calls_of_many_rows(tmp_path):
    """More rows than one tile of the tcgen05 GEMM holds (256): the dense projections run as row chunks of one launch, the
    last chunk partly filled; two prompts of unequal length in one call, against the oracle and against portions that
    each fit a single tile."""
    every = dict(experts=4, top=4, groups=2, keep=2, ff=64, shared_ff=64)
    cfg = U.config([U.wkv(heads=2, dim=32, rank=64, mlp=U.moe(**every)), U.latent(heads=2, dim=32, rot_dim=16, vdim=32, kv_rank=64, q_rank=64),
                    U.mlstm(heads=2, dim=32, vdim=64, mlp=U.moe(**every))], width=128, vocab=96)
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
    plain = PlainModel(cfg, tensors)
    prompts = [_tokens(n, cfg["vocab"], 70 + i) for i, n in enumerate([21, 5, 40])]
    llm = LLM(path, dtype="float32", kvcache_block_size=16, max_model_len=128, max_num_batched_tokens=128, max_num_seqs=2)
    try:
        outs, _ = llm.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=12, ignore_eos=True), use_tqdm=False)
    finally:
        llm.exit()
    for p, o in zip(prompts, outs):
        assert o["token_ids"] == plain.greedy(p, 12)
