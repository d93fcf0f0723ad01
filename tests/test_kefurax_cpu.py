"""Host side of the Kefurax family without a GPU: registry, config reader, weight packing, and the plain oracle's own
invariants (a prompt fed whole, in portions or token by token gives the same logits)."""
import json

import numpy as np
import torch

from tests import kefurax_plain as P
from tests import kefurax_util as U

LAYERS = [U.rglru(mlp=U.dense()), U.parallel(mlp=U.dense(16)), U.mamba1(), U.parallel(left=U.attention(heads=3, kv_heads=1, dim=6, vdim=9, dims=6, scaling=None),
                                                                                   right=U.delta(heads=2, kv_heads=1, dim=7, vdim=4, conv=2))]


def test_registry_and_config_reader(tmp_path):
    from ssd_b200.config import load_hf_config
    from ssd_b200.hybrid import HybridSpec
    from ssd_b200 import lib as L
    cfg = U.config(LAYERS, width=36, vocab=44, mult=0.25, embed_scale=3.5)
    path = U.write_checkpoint(str(tmp_path / "m"), cfg, U.random_tensors(cfg))
    hf = load_hf_config(path)
    assert hf.family.name == "kefurax" and hf.family.kind == "hybrid"
    s = HybridSpec.from_dir(path)
    assert (s.width, s.vocab, s.eps, s.embed_scale, s.residual_mult) == (36, 44, 1e-5, 3.5, 0.25)
    assert s.block == L.BLOCK_SERIAL_POSTNORM and s.norm_offset == 0.0 and s.has_cache and s.has_state
    r, a, m, b = s.layers
    assert (r.mixer, r.inner, r.blocks, r.conv, r.mlp, r.ff, r.decay_mult) == ("rglru", 24, 2, 4, "dense", 24, 8.0)
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.rot_dims, a.qk_norm, a.sink) == (4, 2, 8, 6, 4, 1, 1.0)
    assert (a.yarn_factor, a.yarn_original, a.yarn_fast, a.yarn_slow) == (4.0, 64.0, 8.0, 1.0)
    assert (a.d_heads, a.d_kv_heads, a.d_dim, a.d_vdim, a.conv, a.left_scale, a.right_scale) == (4, 2, 6, 5, 3, 0.7, 1.2)
    assert (m.mixer, m.inner, m.state, m.dt_rank, m.conv, m.mlp) == ("mamba1", 20, 6, 3, 3, None)
    assert b.yarn_factor == 0.0 and b.rot_dims == 6 and b.kv_heads == 1
    # a design lists only its own mixers
    bad = json.loads(json.dumps(cfg))
    bad["layers"][0]["type"] = "wkv"
    try:
        HybridSpec.from_config(bad)
        raise AssertionError("accepted a mixer of another design")
    except ValueError:
        pass


def test_weight_packing_shapes(tmp_path):
    from ssd_b200.hybrid import HybridSpec, pack_hybrid_weights
    cfg = U.config(LAYERS)
    t = U.random_tensors(cfg)
    w = pack_hybrid_weights(HybridSpec.from_config(cfg), t, torch.float32, "cpu")
    r, a, m, _ = w["layers"]
    assert r["RGLRU_IN"].shape == (48, 40) and r["RGLRU_GATE"].shape == (2, 24, 12) and r["GLU_IN"].shape == (48, 40)
    assert torch.equal(r["RGLRU_GATE"][1, 12:], t["l0.mix.ri"][1]) and torch.equal(r["RGLRU_IN_B"][24:], t["l0.mix.x.b"])
    n_left, n_right = 4 * 8 + 2 * 8 + 2 * 6 + 4 * 6, 2 * 2 * 6 + 4 * 5 + 4 * 5 + 4 + 4
    assert a["PAIR_IN"].shape == (n_left + n_right, 40) and a["CONV_W"].shape == (2 * 2 * 6 + 4 * 5, 3)
    assert torch.equal(a["PAIR_IN"][n_left + 12:n_left + 24], t["l1.mix.right.k"])
    assert torch.equal(a["MIX_NORM"].view(4, 5)[3], t["l1.mix.right.norm"])
    assert m["SEL_X"].shape == (3 + 12, 20) and "NORM2" not in m


def test_oracle_portions_equal_whole():
    cfg = U.config(LAYERS)
    plain = U.PlainModel(cfg, U.random_tensors(cfg, 1))
    toks = torch.randint(0, 50, (40,), generator=torch.Generator().manual_seed(2)).tolist()
    whole = plain.run(toks)
    for sizes in ([1] * 40, [2, 3, 1, 7, 2, 25]):
        st, pos, out = {}, 0, []
        for c in sizes:
            out.append(plain.run(toks[pos:pos + c], state=st, p0=pos))
            pos += c
        assert torch.allclose(torch.cat(out), whole, rtol=1e-9, atol=1e-9)


def test_oracle_mechanisms():
    # the convolution's last column meets the current token; zeros come before the sequence
    w = torch.tensor([[0.0, 0.0, 1.0], [1.0, 0.0, 0.0]], dtype=P.F64)
    u = torch.arange(1, 9, dtype=P.F64).view(4, 2)
    out = P.short_conv(u, w, None, {}, "c")
    assert out[:, 0].tolist() == [1.0, 3.0, 5.0, 7.0] and out[:, 1].tolist() == [0.0, 0.0, 2.0, 4.0]
    # frequency scaling: fast dimensions keep their frequency, slow ones are divided by the factor
    rot = {"base": 5000.0, "dims": 24, "scaling": {"factor": 5.0, "original": 300, "fast": 20.0, "slow": 2.0}}
    f, mult = P.rotary_table(rot)
    plain_f = torch.tensor([5000.0 ** (-2.0 * i / 24) for i in range(12)], dtype=P.F64)
    assert abs(f[0] - plain_f[0]) < 1e-15 and abs(f[-1] - plain_f[-1] / 5.0) < 1e-15 and abs(mult - (0.1 * np.log(5.0) + 1.0)) < 1e-12
    assert all(f[i] <= plain_f[i] + 1e-18 for i in range(12))
    # the sink takes a share of the weight: with one key of score 0 the output is half the value
    Wt = {"a.q": torch.zeros(2, 2, dtype=P.F64), "a.k": torch.zeros(2, 2, dtype=P.F64), "a.v": torch.eye(2, dtype=P.F64),
          "a.g": torch.zeros(2, 2, dtype=P.F64), "a.o": torch.eye(2, dtype=P.F64)}
    o = P.sink_attention(torch.tensor([[2.0, 4.0]], dtype=P.F64), Wt, "a", {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 2, "scale": 1.0},
                         1e-6, {}, 0)
    assert torch.allclose(o, torch.tensor([[0.5, 1.0]], dtype=P.F64))  # (value / 2) * sigmoid(0)
