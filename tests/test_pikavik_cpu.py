"""Host side of the hybrid family, no GPU: registry and configuration reading, checkpoint packing, the state-slot pool,
page / slot reuse through Scheduler.extend / release, and the oracle's own consistency (portions == whole)."""
import json
import os

import pytest
import torch

from tests import pikavik_util as U
from tests.pikavik_plain import PlainModel


def _ckpt(tmp_path, layers, seed=0, **kw):
    cfg = U.config(layers, **kw)
    tensors = U.random_tensors(cfg, seed)
    return cfg, tensors, U.write_checkpoint(str(tmp_path / "ckpt"), cfg, tensors)


def test_registry_picks_the_family_from_config_json(tmp_path):
    from ssd_b200.config import load_hf_config
    from ssd_b200.registry import family_of
    _, _, path = _ckpt(tmp_path, [U.wkv()])
    hf = load_hf_config(path)
    assert hf.family.name == "pikavik" and hf.family.kind == "hybrid" and hf.vocab_size == 50
    assert family_of({"model_type": "llama", "hidden_size": 64}).kind == "dense"
    assert family_of({"model_type": "qwen3", "hidden_size": 64}).name == "qwen3"
    with pytest.raises(ValueError):
        family_of({"architecture": "SomethingElse"})


def test_spec_reads_every_size_from_config_and_shapes(tmp_path):
    from ssd_b200.hybrid import HybridSpec
    layers = [U.wkv(heads=3, dim=20, rank=5, mlp=U.moe(experts=8, top=4, groups=2, keep=2, ff=24, shared_ff=0)),
              U.mlstm(heads=1, dim=33, vdim=7, cap=3.0), U.latent(heads=5, dim=4, rot_dim=12, vdim=3, kv_rank=7, q_rank=30, scale=0.7, base=50.0)]
    _, _, path = _ckpt(tmp_path, layers, width=24, vocab=31, eps=1e-5)
    s = HybridSpec.from_dir(path)
    assert (s.width, s.vocab, s.eps, len(s.layers)) == (24, 31, 1e-5, 3)
    a, b, c = s.layers
    assert (a.mixer, a.heads, a.dim, a.decay_rank, a.experts, a.top, a.groups, a.keep, a.ff, a.shared_ff) == ("wkv", 3, 20, 5, 8, 4, 2, 2, 24, 0)
    assert (b.mixer, b.heads, b.dim, b.vdim, b.gate_cap, b.mlp) == ("mlstm", 1, 33, 7, 3.0, None)
    assert (c.heads, c.dim, c.rot_dim, c.rot_dims, c.vdim, c.kv_rank, c.q_rank, c.attn_scale, c.rot_base) == (5, 4, 12, 12, 3, 7, 30, 0.7, 50.0)
    assert s.has_latent and s.has_state


def test_packing_matches_the_bound_layout(tmp_path):
    from ssd_b200.hybrid import HybridSpec, pack_hybrid_weights, read_safetensors
    cfg, tensors, path = _ckpt(tmp_path, [U.wkv(mlp=U.moe()), U.mlstm(), U.latent()])
    raw = read_safetensors(os.path.join(path, "model.safetensors"))
    assert set(raw) == set(tensors) and all(torch.equal(raw[k].float(), tensors[k]) for k in raw)
    w = pack_hybrid_weights(HybridSpec.from_dir(path), raw, torch.float32, "cpu")
    l0, l1, l2 = w["layers"]
    assert l0["WKV_MU"].shape == (5, 40) and torch.equal(l0["WKV_MU"][4], tensors["l0.mix.mu.w"])
    assert l0["EXPERT_IN"].shape == (6, 40, 40) and torch.equal(l0["EXPERT_IN"][2, 20:], tensors["l0.mlp.e2.up"])
    assert l0["SHARED_IN"].shape == (25, 40) and torch.equal(l0["SHARED_IN"][24], tensors["l0.mlp.shared.sg"][0])
    assert l1["MLSTM_IN"].shape == (2 * 20 + 2 * 12 + 4, 40) and torch.equal(l1["MLSTM_IN"][-2:], tensors["l1.mix.f"])
    uk = tensors["l2.mix.uk"].view(3, 10, 20)
    assert l2["LAT_UKT"].shape == (3, 20, 10) and torch.equal(l2["LAT_UKT"][1], uk[1].T)
    assert torch.equal(l2["LAT_DOWN"][18:], tensors["l2.mix.dkv"])


def test_state_slots_and_pages_go_round(tmp_path, monkeypatch):
    from ssd_b200.config import Config
    from ssd_b200.engine.scheduler import Scheduler
    from ssd_b200.engine.sequence import Sequence
    from ssd_b200.engine.state_manager import StateSlotManager
    _, _, path = _ckpt(tmp_path, [U.wkv(), U.latent()])
    cfg = Config(path, kvcache_block_size=16, num_kvcache_blocks=5, max_model_len=80, max_num_batched_tokens=80, max_num_seqs=2)
    monkeypatch.setattr(Sequence, "block_size", 16)
    sm = StateSlotManager(2)
    sched = Scheduler(cfg, state_manager=sm, prefix_reuse=False)
    a, b, c = Sequence([]), Sequence([]), Sequence([])
    assert sched.extend(a, list(range(20))) == 0 and a.state_slot == 0 and a.block_table == [0, 1]
    assert sched.extend(b, list(range(16))) == 0 and b.state_slot == 1 and b.block_table == [2]
    assert sched.extend(a, list(range(13))) == 20 and a.block_table == [0, 1, 3]      # 33 tokens: a third page
    with pytest.raises(RuntimeError):
        sched.extend(c, [1, 2, 3])                                                    # no slot left
    assert sched.extend(b, [7]) == 16 and b.block_table == [2, 4]
    with pytest.raises(RuntimeError):
        sched.extend(a, list(range(16)))                                              # no page left
    sched.release(a)
    assert a.state_slot == -1 and a.block_table == [] and sm.can_allocate()
    assert sched.extend(c, list(range(40))) == 0 and c.state_slot == 0 and sorted(c.block_table) == [0, 1, 3]
    # identical prompts never share pages in a model with recurrent state
    sched.release(b)
    d = Sequence([])
    sched.extend(d, list(range(16)))
    assert not set(d.block_table) & set(c.block_table) and d.num_cached_tokens == 0
    sched.release(c); sched.release(d)
    assert len(sched.block_manager.free_block_ids) == 5 and len(sm.free_slots) == 2 and sched.is_finished()


def test_hybrid_config_limits(tmp_path):
    from ssd_b200.config import Config
    _, _, path = _ckpt(tmp_path, [U.mlstm()])
    with pytest.raises(NotImplementedError):
        Config(path, speculate=True, draft=path)
    with pytest.raises(ValueError):
        Config(path, dtype="float16")
    assert Config(path, dtype="float32").family.kind == "hybrid"


def test_oracle_portions_equal_whole():
    cfg = U.config([U.mlstm(mlp=U.moe()), U.wkv(), U.latent(mlp=U.moe(experts=4, top=1, groups=1, keep=1, shared_ff=0))])
    m = PlainModel(cfg, U.random_tensors(cfg, 5))
    toks = torch.randint(0, 50, (45,), generator=torch.Generator().manual_seed(1)).tolist()
    whole = m.run(toks)
    st, out, pos = m.new_state(), [], 0
    for c in (2, 17, 1, 25):
        out.append(m.run(toks[pos:pos + c], st, pos))
        pos += c
    assert torch.allclose(torch.cat(out), whole, rtol=0, atol=1e-10)


def test_oracle_routing_by_hand():
    from tests.pikavik_plain import route
    s = torch.tensor([0.9, 0.1, 0.5, 0.6, 0.8, 0.3], dtype=torch.float64)   # groups of two: sums 1.0, 1.1, 1.1
    chosen, w = route(s, top=2, groups=3, keep=2, scale=2.0)                 # groups 1 and 2 stay (tie: lower first)
    assert chosen == [4, 3] and torch.allclose(w, torch.tensor([0.8, 0.6], dtype=torch.float64) / 1.4 * 2.0)
    chosen, _ = route(s, top=3, groups=1, keep=1, scale=1.0)
    assert chosen == [0, 4, 3]
