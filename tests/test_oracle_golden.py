"""The CPU oracle against its pins: gguf-py decode vectors, the reference's
routing known-answer cases (src/moe.rs:405-484), and internal consistency."""
import json
import os

import numpy as np

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def test_decode_matches_gguf_py(orc):
    z = np.load(os.path.join(GOLD, "kquant_decode.npz"))
    for name, dt in (("q4k", orc.Q4_K), ("q6k", orc.Q6_K)):
        blocks, want = z[name + "_blocks"], z[name + "_decoded"]
        got = orc.dequantize(dt, blocks).reshape(want.shape)
        # gguf-py evaluates (d*sc)*q - dmin*m in float32 like the oracle; allow 1 ulp-ish
        np.testing.assert_allclose(got, want, rtol=2e-6, atol=1e-9)


def test_routing_known_answers(orc):
    cases = json.load(open(os.path.join(GOLD, "routing_kat.json")))
    assert len(cases) == 4
    for c in cases:
        ids, w = orc.route_from_logits(np.array([c["logits"]], np.float32), np.array(c["bias"], np.float32),
                                       c["top_k"], c["scale"], c["norm"])
        assert ids[0].tolist() == c["ids"], c["name"]
        want = np.array(c["weights"])
        tol = c["atol"] + c["rtol"] * np.abs(want)
        assert np.all(np.abs(w[0] - want) <= tol), (c["name"], w[0], want)


def test_router_matmul_matches_direct_logits(orc):
    # identity router: logits == x (src/moe.rs:486-500)
    x = np.array([[2.0, -2.0, 0.0, 1.0, -1.0, 3.0, 0.5, -0.5]], np.float32)
    got = orc.route_logits(np.eye(8, dtype=np.float32), x)
    np.testing.assert_allclose(got, x, atol=1e-6)


def test_sigmoid_accuracy(orc):
    v = np.linspace(-30, 30, 2001).astype(np.float32)
    got = np.array([orc.lib().lmo_sigmoid(float(a)) for a in v])
    want = 1.0 / (1.0 + np.exp(-v.astype(np.float64)))
    assert np.max(np.abs(got - want) / want) < 4e-7


def test_router_dot_close_to_f64(orc):
    rng = np.random.default_rng(0)
    r = (rng.standard_normal((16, 3072)) * 0.02).astype(np.float32)
    x = rng.standard_normal((3, 3072)).astype(np.float32)
    got = orc.route_logits(r, x)
    want = x.astype(np.float64) @ r.astype(np.float64).T
    assert np.max(np.abs(got - want)) < 2e-6


def test_encoder_roundtrip_error(orc):
    rng = np.random.default_rng(1)
    w = (rng.standard_normal(64 * 256) * 0.02).astype(np.float32)
    for dt, bound in ((orc.Q4_K, 0.08), (orc.Q6_K, 0.02)):
        deq = orc.dequantize(dt, orc.quantize(dt, w))
        assert orc.rel_l2(deq, w) < bound
    # all-zero block stays zero
    for dt in (orc.Q4_K, orc.Q6_K):
        assert np.all(orc.dequantize(dt, orc.quantize(dt, np.zeros(256, np.float32))) == 0)


def test_mul_id_against_numpy(orc):
    # testutil::oracle shape (src/ops/dispatch.rs:2273-2300): shared row and per-slot rows
    for dt in (orc.Q4_K, orc.Q6_K):
        ne, n_out, k, t, top_k = 4, 8, 512, 3, 2
        w = orc.pseudo_random(ne * n_out * k, 0x100, -1.0, 1.0)
        stack = orc.quantize(dt, w)
        deq = orc.dequantize(dt, stack).reshape(ne, n_out, k).astype(np.float64)
        ids = orc.random_ids(t, top_k, ne, 0x11)
        for xpr in (1, top_k):
            x = orc.pseudo_random(t * xpr * k, 0xABCD, -1.0, 1.0).reshape(t, xpr, k)
            got = orc.mul_id(dt, stack, ne, n_out, k, x, ids)
            want = np.stack([np.stack([deq[ids[i, s]] @ x[i, 0 if xpr == 1 else s].astype(np.float64)
                                       for s in range(top_k)]) for i in range(t)])
            assert orc.rel_l2(got, want) < 1e-6


def test_map0(orc):
    ids = orc.distinct_ids(40, 4, 6, 0x43)
    tpe, m = orc.map0(ids, 6)
    assert tpe.sum() == 40 * 4
    for e in range(6):
        want = [t * 4 + s for t in range(40) for s in range(4) if ids[t, s] == e]
        assert m[e, : tpe[e]].tolist() == want


def test_combine_and_silu(orc):
    rng = np.random.default_rng(2)
    down = rng.standard_normal((5, 10, 64)).astype(np.float32)
    w = rng.uniform(0, 1, (5, 10)).astype(np.float32)
    l2 = rng.uniform(0.5, 2, (5, 10, 1)).astype(np.float32)
    np.testing.assert_allclose(orc.combine(down, None, w), (down * w[:, :, None]).sum(1), rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(orc.combine(down, l2, w), (down * l2 * 2.0 ** -15 * w[:, :, None]).sum(1),
                               rtol=1e-5, atol=1e-9)
    g, u = down[0], down[1]
    np.testing.assert_allclose(orc.silu_mul(g, u), g / (1 + np.exp(-g)) * u, rtol=1e-6, atol=1e-7)


def _tiny_layer(orc, seed=3, hidden=256, ff=256, ne=4, top_k=2, shared=True):
    rng = np.random.default_rng(seed)
    q = lambda dt, shape: orc.quantize(dt, (rng.uniform(-0.5, 0.5, shape)).astype(np.float32))
    return orc.HostLayer(hidden, ff, ne, top_k,
                         router=(rng.standard_normal((ne, hidden)) * 0.1).astype(np.float32),
                         bias=rng.uniform(-0.1, 0.1, ne).astype(np.float32),
                         gate=q(orc.Q4_K, (ne, ff, hidden)), up=q(orc.Q4_K, (ne, ff, hidden)),
                         down=q(orc.Q6_K, (ne, hidden, ff)),
                         sh_gate=q(orc.Q4_K, (ff, hidden)) if shared else None,
                         sh_up=q(orc.Q4_K, (ff, hidden)) if shared else None,
                         sh_down=q(orc.Q6_K, (hidden, ff)) if shared else None)


def test_moe_block_against_dequantize_everything(orc):
    # the shape of check_reference_experts (src/moe.rs:522-589), tol 1e-3*max(|e|,1)
    L = _tiny_layer(orc)
    rng = np.random.default_rng(4)
    x = rng.uniform(-1, 1, (3, L.hidden)).astype(np.float32)
    out, ids, w = L.forward(x)
    H, F = L.hidden, L.expert_ff
    g = orc.dequantize(orc.Q4_K, L.gate).reshape(-1, F, H).astype(np.float64)
    u = orc.dequantize(orc.Q4_K, L.up).reshape(-1, F, H).astype(np.float64)
    d = orc.dequantize(orc.Q6_K, L.down).reshape(-1, H, F).astype(np.float64)
    sg = orc.dequantize(orc.Q4_K, L.sh_gate).reshape(F, H).astype(np.float64)
    su = orc.dequantize(orc.Q4_K, L.sh_up).reshape(F, H).astype(np.float64)
    sd = orc.dequantize(orc.Q6_K, L.sh_down).reshape(H, F).astype(np.float64)
    ffn = lambda G, U, D, v: D @ ((lambda a: a / (1 + np.exp(-a)))(G @ v) * (U @ v))
    for t in range(3):
        want = ffn(sg, su, sd, x[t].astype(np.float64))
        for s in range(L.top_k):
            e = ids[t, s]
            want = want + w[t, s] * ffn(g[e], u[e], d[e], x[t].astype(np.float64))
        assert np.all(np.abs(out[t] - want) <= 1e-3 * np.maximum(np.abs(want), 1.0))
    out64, ids64, _ = L.forward(x, accum64=True)
    assert np.array_equal(ids, ids64)
    assert orc.rel_l2(out, out64) < 1e-5


def test_q8_baseline_deviation_is_reported_not_gated(orc):
    L = _tiny_layer(orc, seed=5)
    x = np.random.default_rng(6).standard_normal((2, L.hidden)).astype(np.float32)
    ref, _, _ = L.forward(x)
    q8 = L.forward_q8(x)
    assert orc.rel_l2(q8, ref) < 0.05  # int8 activations: percent-level, by construction
