"""The GGUF-fed path: a synthetic qwen3moe-style file written with gguf-py holds one block's MoE-FFN tensors
(Q4_K gate/up, Q4_K or Q6_K down, bf16 router, f32 norm); this repository's reader must locate exactly the bytes
gguf-py hands out for the same names (the offset check of tools/q4k_job.py:51-68), and the decode layer fed from
the file must match the CPU restatement fed from the same arrays."""
import numpy as np
import pytest

import oracle_lib as ol
from kanjoos_b200 import gguf_bank, synth

gguf = pytest.importorskip("gguf")

E, H, F, K = 8, 512, 256, 2


def write_file(path, down_q6k=False):
    bank = synth.expert_bank(501, n_experts=E, hidden=H, ffn=F)
    wr, _ = synth.router_weight(501, n_experts=E, hidden=H)
    rng = np.random.Generator(np.random.Philox(501))
    down = bank["down"]
    if down_q6k:
        down = rng.integers(0, 256, size=(E, H, F // 256, 210), dtype=np.uint8)
        down[..., 208:210] = (np.abs(rng.standard_normal((E, H, F // 256, 1))) * 0.01).astype(np.float16).view(np.uint8)
    norm = (1.0 + 0.02 * rng.standard_normal(H)).astype(np.float32)
    w = gguf.GGUFWriter(str(path), "qwen3moe")
    w.add_block_count(1)
    w.add_embedding_length(H)
    w.add_expert_feed_forward_length(F)
    w.add_expert_count(E)
    w.add_expert_used_count(K)
    w.add_layer_norm_rms_eps(1e-6)
    q4, q6, bf = gguf.GGMLQuantizationType.Q4_K, gguf.GGMLQuantizationType.Q6_K, gguf.GGMLQuantizationType.BF16
    w.add_tensor("blk.0.ffn_norm.weight", norm)
    w.add_tensor("blk.0.ffn_gate_inp.weight", np.ascontiguousarray(wr).view(np.uint8).reshape(E, H * 2), raw_dtype=bf)
    w.add_tensor("blk.0.ffn_gate_exps.weight", bank["gate"].reshape(E, F, -1), raw_dtype=q4)
    w.add_tensor("blk.0.ffn_up_exps.weight", bank["up"].reshape(E, F, -1), raw_dtype=q4)
    w.add_tensor("blk.0.ffn_down_exps.weight", down.reshape(E, H, -1), raw_dtype=q6 if down_q6k else q4)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    return bank, wr, down, norm


@pytest.mark.parametrize("down_q6k", [False, True])
def test_reader_locates_the_tensors(tmp_path, down_q6k):
    path = tmp_path / "synthetic.gguf"
    bank, wr, down, norm = write_file(path, down_q6k)
    g = gguf_bank.GgufFile(str(path))
    assert g.arch() == "qwen3moe" and g.n_layers() == 1
    assert g.meta_int("qwen3moe.expert_count") == E and g.meta_int("qwen3moe.expert_used_count") == K
    assert g.require("blk.0.ffn_gate_exps.weight").dims == (H, F, E)   # ggml order: input dimension first
    assert g.require("blk.0.ffn_down_exps.weight").dims == (F, H, E)
    assert gguf_bank.verify_against_gguf_py(str(path)) == 5
    a = gguf_bank.layer_arrays(g, 0)
    assert np.array_equal(a["gate"], bank["gate"]) and np.array_equal(a["up"], bank["up"])
    assert np.array_equal(a["down"], down) and a["down"].shape[-1] == (210 if down_q6k else 144)
    assert np.array_equal(a["router"], wr) and a["router_exact"] and a["top_k"] == K
    # f32 norm weights are rounded to bf16 for the kernels, to nearest even
    back = (a["norm"].astype(np.uint32) << 16).view(np.float32)
    assert not a["norm_exact"] and np.max(np.abs(back - norm)) <= 2.0 ** -8


def test_missing_tensor_and_bad_magic(tmp_path):
    path = tmp_path / "synthetic.gguf"
    write_file(path)
    g = gguf_bank.GgufFile(str(path))
    with pytest.raises(KeyError):
        g.require("blk.0.attn_q.weight")
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGML" + bytes(60))
    with pytest.raises(ValueError):
        gguf_bank.GgufFile(str(bad))


@pytest.mark.gpu
def test_decode_layer_fed_from_the_file(tmp_path):
    import torch
    from gpu_util import report
    from kanjoos_b200.moe import MoeFfnLayer
    path = tmp_path / "synthetic.gguf"
    bank, wr, _, _ = write_file(path)
    g = gguf_bank.GgufFile(str(path))
    eb, top_k = gguf_bank.load_expert_bank(g, 0)
    hx = synth.hidden_rows(501, 5, H)
    want, _, _ = ol.moe(wr, bank, hx, K)
    layer = MoeFfnLayer(eb, top_k=top_k, max_tokens=5, use_norm=False)
    got = layer.decode(torch.from_numpy(hx).cuda()).cpu().numpy()
    st = report(got, want, "decode layer fed from a GGUF file")
    assert st["rel_rmse"] <= 1e-5
