"""CPU: the checkpoint converter (GPTQ-style 4-bit state dict -> packed 2:4 tensors keyed
{module}.{tp}.{qweight,scales,meta}) against vectors made by the reference's own dequantiser and
tensor-parallel packer, and against the oracle decoder."""
import os

import numpy as np
import pytest
import torch

from oracle import delta_format as fmt

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_vectors.npz"))


def test_gptq_dequantize_matches_reference_vector():
    from triteia_b200.utils.quant_utils import dequantize_weight

    got = dequantize_weight(torch.from_numpy(GOLD["gptq_qweight"]), torch.from_numpy(GOLD["gptq_qzeros"]),
                            torch.from_numpy(GOLD["gptq_scales"]))
    assert got.dtype == torch.float16 and np.array_equal(got.numpy(), GOLD["gptq_dense"])


def test_asymmetric_checkpoint_is_refused():
    from triteia_b200.utils.quant_utils import dequantize_weight

    z = torch.from_numpy(GOLD["gptq_qzeros"]).clone()
    z[0, 0] = 0x77777776
    with pytest.raises(ValueError):
        dequantize_weight(torch.from_numpy(GOLD["gptq_qweight"]), z, torch.from_numpy(GOLD["gptq_scales"]))


@pytest.mark.parametrize("how", ["column", "row"])
def test_tensor_parallel_chunks_match_reference_vectors(how):
    from triteia_b200.ops.utils.generator import torch_weight_to_sparse_marlin

    qs, ss, ms = torch_weight_to_sparse_marlin(torch.from_numpy(GOLD["tp_weight"]), torch.from_numpy(GOLD["tp_scale"]),
                                               tp_size=2, chunk_by=how)
    for i in range(2):
        assert np.array_equal(qs[i].numpy(), GOLD[f"tp_{how}_{i}_q"])
        assert np.array_equal(ss[i].numpy(), GOLD[f"tp_{how}_{i}_s"])
        assert np.array_equal(ms[i].numpy(), GOLD[f"tp_{how}_{i}_meta"])


def _gptq_module(rng, k, n):
    """A symmetric 4-bit module whose dense weight is 2:4 sparse along the input features: code 8 is
    level 0 (zero point 7 + 1), kept positions carry a non-zero level."""
    lev = rng.integers(1, 8, (k, n)) * (rng.integers(0, 2, (k, n)) * 2 - 1)
    keep = rng.random((k // 4, 4, n)).argsort(axis=1).argsort(axis=1) < 2        # two of every four rows
    codes = (lev * keep.reshape(k, n) + 8).astype(np.int64)                      # [in, out]
    q = np.zeros((k // 8, n), dtype=np.int64)
    for i in range(8):
        q |= codes[i::8] << (4 * i)
    q = q.astype(np.uint32).view(np.int32)
    scales = (rng.random((1, n)) * 0.01 + 0.001).astype(np.float16)
    dense = ((codes - 8) * scales.astype(np.float32)).astype(np.float16)         # [in, out]
    return {"qweight": torch.from_numpy(q), "qzeros": torch.full((1, n // 8), 0x77777777, dtype=torch.int32),
            "scales": torch.from_numpy(scales), "g_idx": torch.zeros(k, dtype=torch.int32)}, dense


@pytest.mark.parametrize("tp", [1, 2])
def test_convert_state_dict_keys_and_contents(tp, tmp_path):
    from triteia_b200.converters.deltazip import convert_model, convert_state_dict

    rng = np.random.default_rng(3)
    hidden, inter = 512, 1024
    shapes = {"self_attn.q_proj": (hidden, hidden), "self_attn.k_proj": (hidden, hidden), "self_attn.v_proj": (hidden, hidden),
              "self_attn.o_proj": (hidden, hidden), "mlp.gate_proj": (hidden, inter), "mlp.up_proj": (hidden, inter),
              "mlp.down_proj": (inter, hidden)}
    tensors, dense = {}, {}
    for name, (k, n) in shapes.items():
        mod, d = _gptq_module(rng, k, n)
        dense[name] = d
        for suffix, t in mod.items():
            tensors[f"model.layers.0.{name}.{suffix}"] = t
    tensors["model.embed_tokens.weight"] = torch.randn(64, hidden).half()
    tensors["lm_head.weight"] = torch.randn(64, hidden).half()
    tensors["model.layers.0.input_layernorm.weight"] = torch.ones(hidden).half()
    out = convert_state_dict(tensors, tp)

    fused = {"self_attn.qkv_proj": np.concatenate([dense["self_attn.q_proj"], dense["self_attn.k_proj"], dense["self_attn.v_proj"]], axis=1),
             "mlp.gate_up_proj": np.concatenate([dense["mlp.gate_proj"], dense["mlp.up_proj"]], axis=1)}
    expect_keys = set()
    for name, w in fused.items():                                   # split by output columns
        for i in range(tp):
            key = f"model.layers.0.{name}.{i}"
            expect_keys |= {key + ".qweight", key + ".scales", key + ".meta"}
            cols = w.shape[1] // tp
            got = fmt.dequantize(out[key + ".qweight"].numpy(), out[key + ".meta"].numpy(), out[key + ".scales"].numpy())
            assert np.array_equal(got.astype(np.float16), w[:, i * cols:(i + 1) * cols])
    for name in ("self_attn.o_proj", "mlp.down_proj"):              # split by input rows
        for i in range(tp):
            key = f"model.layers.0.{name}.{i}"
            expect_keys |= {key + ".qweight", key + ".scales", key + ".meta"}
            rows = dense[name].shape[0] // tp
            got = fmt.dequantize(out[key + ".qweight"].numpy(), out[key + ".meta"].numpy(), out[key + ".scales"].numpy())
            assert np.array_equal(got.astype(np.float16), dense[name][i * rows:(i + 1) * rows])
    for name in ("model.embed_tokens", "lm_head"):
        for i in range(tp):
            expect_keys.add(f"{name}.{i}.weight")
            assert torch.equal(out[f"{name}.{i}.weight"], tensors[name + ".weight"][i * 64 // tp:(i + 1) * 64 // tp])
    assert set(out) == expect_keys                                  # nothing else is carried over

    # the file form: safetensors in, safetensors out
    from safetensors.torch import load_file, save_file
    src, dst = str(tmp_path / "in.safetensors"), str(tmp_path / "out.safetensors")
    save_file({k: v.contiguous() for k, v in tensors.items()}, src)
    convert_model(src, tp, dst)
    back = load_file(dst)
    assert set(back) == expect_keys and all(torch.equal(back[k], out[k].contiguous()) for k in back)
