"""GGUF container reader: files written by the `gguf` package (an independent implementation of the
format) are parsed, the quantized stacks come back byte for byte, and a block loaded from a file gives
the oracle's result on the GPU."""
import numpy as np
import pytest
import torch

gguf = pytest.importorskip("gguf")

H, F, E, K = 256, 256, 8, 3


def _write(path, orc, seed=5, shared=True, bias_suffix="bias"):
    rng = np.random.default_rng(seed)
    q = lambda dt, shape: orc.quantize(dt, rng.uniform(-0.5, 0.5, shape).astype(np.float32))
    t = {
        "router": (rng.standard_normal((E, H)) * 0.1).astype(np.float32),
        "bias": rng.uniform(-0.1, 0.1, E).astype(np.float32),
        "gate": q(orc.Q4_K, (E, F, H)), "up": q(orc.Q4_K, (E, F, H)), "down": q(orc.Q6_K, (E, H, F)),
        "sh_gate": q(orc.Q4_K, (F, H)), "sh_up": q(orc.Q4_K, (F, H)), "sh_down": q(orc.Q6_K, (H, F)),
        "norm": rng.uniform(0.5, 1.5, H).astype(np.float32),
    }
    w = gguf.GGUFWriter(str(path), "laguna")
    w.add_uint32("laguna.expert_used_count", K)
    w.add_float32("laguna.expert_weights_scale", 2.5)
    w.add_bool("laguna.expert_weights_norm", True)
    w.add_array("tokenizer.dummy", ["a", "b"])          # a string array the reader has to step over
    Q4, Q6 = gguf.GGMLQuantizationType.Q4_K, gguf.GGMLQuantizationType.Q6_K
    raw = lambda a, shape, per: np.asarray(a, np.uint8).reshape(*shape[:-1], shape[-1] // 256 * per)
    w.add_tensor("blk.2.ffn_gate_inp.weight", t["router"])
    w.add_tensor(f"blk.2.exp_probs_b.{bias_suffix}", t["bias"])
    w.add_tensor("blk.2.ffn_norm.weight", t["norm"])
    w.add_tensor("blk.2.ffn_gate_exps.weight", raw(t["gate"], (E, F, H), 144), raw_dtype=Q4)
    w.add_tensor("blk.2.ffn_up_exps.weight", raw(t["up"], (E, F, H), 144), raw_dtype=Q4)
    w.add_tensor("blk.2.ffn_down_exps.weight", raw(t["down"], (E, H, F), 210), raw_dtype=Q6)
    if shared:
        w.add_tensor("blk.2.ffn_gate_shexp.weight", raw(t["sh_gate"], (F, H), 144), raw_dtype=Q4)
        w.add_tensor("blk.2.ffn_up_shexp.weight", raw(t["sh_up"], (F, H), 144), raw_dtype=Q4)
        w.add_tensor("blk.2.ffn_down_shexp.weight", raw(t["sh_down"], (H, F), 210), raw_dtype=Q6)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    return t


def test_directory_and_raw_bytes(orc, tmp_path):
    from maxuna_b200.gguf_file import GgufError, GgufFile

    orc.build()
    t = _write(tmp_path / "m.gguf", orc)
    g = GgufFile(str(tmp_path / "m.gguf"))
    assert g.version == 3 and g.kv["general.architecture"] == "laguna"
    assert g.moe_config() == {"n_expert_used": K, "weights_scale": 2.5, "weights_norm": True, "rms_eps": 1e-6}
    i = g.info("blk.2.ffn_down_exps.weight")
    assert i.shape == (E, H, F) and i.ggml_type == 14 and i.nbytes == E * H * (F // 256) * 210
    assert g.info("blk.2.ffn_gate_shexp.weight").shape == (F, H)
    for name, key in (("ffn_gate_exps", "gate"), ("ffn_up_exps", "up"), ("ffn_down_exps", "down"),
                      ("ffn_down_shexp", "sh_down")):
        assert np.array_equal(g.raw(f"blk.2.{name}.weight"), np.asarray(t[key], np.uint8).reshape(-1))
        assert (g.data_offset + g.info(f"blk.2.{name}.weight").offset) % 32 == 0     # src/gguf.rs:111-113
    assert torch.equal(g.f32("blk.2.ffn_gate_inp.weight"), torch.from_numpy(t["router"]))
    assert torch.equal(g.ffn_norm(2, "cpu"), torch.from_numpy(t["norm"]))
    with pytest.raises(GgufError, match="not found"):
        g.info("blk.9.ffn_gate_exps.weight")
    with pytest.raises(GgufError, match="F32/F16"):
        g.f32("blk.2.ffn_gate_exps.weight")
    with pytest.raises(GgufError, match="no fused kernels"):
        g.expert_stack("blk.2.ffn_gate_inp.weight", device="cpu")
    g.close()


def test_malformed_files(tmp_path):
    from maxuna_b200.gguf_file import GgufError, GgufFile

    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGML" + b"\0" * 64)
    with pytest.raises(GgufError, match="not a GGUF"):
        GgufFile(str(bad))
    bad.write_bytes(b"GGUF" + (1).to_bytes(4, "little") + b"\0" * 16)
    with pytest.raises(GgufError, match="version 1"):
        GgufFile(str(bad))
    bad.write_bytes(b"GGUF" + (3).to_bytes(4, "little") + (5).to_bytes(8, "little") + (0).to_bytes(8, "little"))
    with pytest.raises(GgufError, match="truncated"):
        GgufFile(str(bad))


@pytest.mark.gpu
@pytest.mark.parametrize("shared,suffix", [(True, "bias"), (False, "weight")])
def test_block_from_file_matches_oracle(orc, tmp_path, shared, suffix):
    from maxuna_b200.gguf_file import GgufFile

    orc.build()
    t = _write(tmp_path / "m.gguf", orc, seed=6, shared=shared, bias_suffix=suffix)
    g = GgufFile(str(tmp_path / "m.gguf"))
    blk = g.moe_block(2, device="cuda:0")
    assert (blk.n_expert, blk.hidden, blk.expert_ff, blk.n_expert_used) == (E, H, F, K)
    host = orc.HostLayer(H, F, E, K, t["router"], t["bias"], t["gate"], t["up"], t["down"],
                         *((t["sh_gate"], t["sh_up"], t["sh_down"]) if shared else ()))
    x = np.random.default_rng(8).standard_normal((5, H)).astype(np.float32)
    out, ids, w = blk.forward(torch.from_numpy(x).cuda(), return_routing=True)
    want, ids_o, w_o = host.forward(x)
    assert np.array_equal(ids.cpu().numpy().astype(np.uint32), ids_o)
    assert orc.rel_l2(out.cpu().numpy(), want) < 2e-3
