"""CPU: the oracle against the vectors produced by the reference's own Python code
(tests/golden/make_golden.py), and the product packer / generators against the same vectors."""
import numpy as np
import pytest
import torch

from oracle import delta_format as fmt
from oracle import ops as oracle
from triteia_b200.ops.utils import generator as gen
from triteia_b200.ops.utils.sparsity import compress_2_4, mask_creator, pack_2_4

PACK_CASES = {"pack_a": (256, 128, 1), "pack_b": (512, 256, 2), "pack_c": (256, 384, 3)}


@pytest.mark.parametrize("name", list(PACK_CASES))
def test_decoder_matches_reference_uncompress(golden, name):
    w = fmt.dequantize(golden[f"{name}_q"], golden[f"{name}_meta"], golden[f"{name}_s"])
    ref = golden[f"{name}_uncompress"]
    assert w.shape == ref.shape and w.dtype == np.float16
    assert np.array_equal(w, ref)  # value-exact (the reference stores -0.0 at some pruned slots)
    nz = ref != 0
    assert np.array_equal(w.view(np.uint16)[nz], ref.view(np.uint16)[nz])


def test_decoder_batched(golden):
    for b in range(golden["sbmm_q"].shape[0]):
        w = fmt.dequantize(golden["sbmm_q"][b], golden["sbmm_meta"][b], golden["sbmm_s"][b])
        assert np.array_equal(w, golden["sbmm_unc"][b])


def test_decoded_matrix_is_2_of_4(golden):
    lev = fmt.dense_levels(golden["pack_b_q"], golden["pack_b_meta"])
    k, n = lev.shape
    assert ((lev.reshape(k // 4, 4, n) != 0).sum(axis=1) <= 2).all()


@pytest.mark.parametrize("name", list(PACK_CASES))
def test_packer_bit_exact_with_reference(golden, name):
    n, k, seed = PACK_CASES[name]
    torch.manual_seed(seed)
    unc, q, s, meta = gen.gen_sparse_quant4_NT(n, k, device="cpu")
    assert np.array_equal(unc.numpy().view(np.uint16), golden[f"{name}_uncompress"].view(np.uint16))
    assert np.array_equal(q.numpy(), golden[f"{name}_q"])
    assert np.array_equal(s.numpy(), golden[f"{name}_s"])
    assert np.array_equal(meta.numpy(), golden[f"{name}_meta"])


def test_compressor_matches_reference(golden):
    sp, me = compress_2_4(torch.from_numpy(golden["comp_dense"]))
    assert np.array_equal(sp.numpy(), golden["comp_sparse"])
    assert np.array_equal(me.numpy(), golden["comp_meta"])


def test_mask_creator(golden):
    m = mask_creator(torch.from_numpy(golden["mask_in"]), 2, 4)
    assert np.array_equal(m.numpy(), golden["mask_out"])
    with pytest.raises(ValueError):
        mask_creator(torch.zeros(3, 3), 2, 4)


def test_index_distributions(golden):
    np.random.seed(5)
    assert np.array_equal(gen.generate_model_distribution("uniform", 64, 8, device="cpu").numpy(), golden["dist_uniform"])
    np.random.seed(5)
    assert np.array_equal(gen.generate_model_distribution("zipf:1.5", 64, 8, device="cpu").numpy(), golden["dist_zipf"])
    z = gen.generate_model_distribution("true-zipf:1.5", 4096, 16, device="cpu", rng=np.random.default_rng(0)).numpy()
    counts = np.bincount(z, minlength=16)
    assert z.min() >= 0 and counts[0] > counts[3] > counts[15]


@pytest.mark.parametrize("case", ["route_a", "route_b", "route_c", "route_d"])
def test_route_matches_reference_prologue(golden, case):
    u, st, c = oracle.route_sorted(golden[f"{case}_idx"])
    assert np.array_equal(u, golden[f"{case}_unique"])
    assert np.array_equal(st, golden[f"{case}_start"])
    assert np.array_equal(c, golden[f"{case}_count"])


def test_route_any_is_stable_sort():
    rng = np.random.default_rng(3)
    idx = rng.integers(-1, 7, size=200).astype(np.int32)
    perm, u, st, c = oracle.route_any(idx)
    assert np.array_equal(np.sort(perm), np.arange(200))
    s = idx[perm]
    assert (np.diff(s) >= 0).all()
    for d, a, n in zip(u, st, c):
        assert (s[a:a + n] == d).all()
        assert (np.diff(perm[a:a + n]) > 0).all()  # stable
    assert c.sum() == (idx >= 0).sum()


def test_sbmm_oracle_vs_reference_fp16_loop(golden):
    y = oracle.sbmm(golden["sbmm_q"], golden["sbmm_x"], golden["sbmm_meta"], golden["sbmm_s"], golden["sbmm_idx"])
    assert oracle.row_rel_err(golden["sbmm_y"], y).max() < 1e-2
    yb = oracle.sbmm(golden["sbmm_q"], golden["sbmm_x"], golden["sbmm_meta"], golden["sbmm_s"], golden["sbmm_idx"],
                     base_weight=golden["sbmm_base"])
    assert oracle.row_rel_err(golden["sbmm_y_base"], yb).max() < 1e-2
    assert np.all(y[golden["sbmm_idx"] == -1] == 0)


def test_lora_and_ldmm_oracle_vs_reference(golden):
    y = oracle.lora(golden["lora_A"], golden["lora_B"], golden["lora_x"], golden["lora_idx"])
    assert oracle.row_rel_err(golden["lora_y"], y).max() < 1e-2
    yd = oracle.ldmm(golden["ldmm_idx"], golden["ldmm_x"], golden["lora_A"], golden["lora_B"], golden["sbmm_q"],
                     golden["sbmm_meta"], golden["sbmm_s"])
    assert oracle.row_rel_err(golden["ldmm_y"], yd).max() < 1e-2


def test_bgmv_sgmv_oracles_agree_with_lora():
    rng = np.random.default_rng(0)
    A = rng.standard_normal((3, 64, 8)).astype(np.float16)
    B = rng.standard_normal((3, 8, 32)).astype(np.float16)
    x = rng.standard_normal((6, 64)).astype(np.float16)
    idx = np.array([0, 0, 1, 2, 2, 2])
    ref = oracle.lora(A, B, x, idx)
    v = oracle.bgmv(np.zeros((6, 8)), x, A.transpose(0, 2, 1)[:, None], idx, 0, 1.0)
    y = oracle.bgmv(np.zeros((6, 32)), v, B.transpose(0, 2, 1)[:, None], idx, 0, 1.0)
    assert np.allclose(y, ref, rtol=1e-5, atol=1e-4)
    seg = np.array([0, 2, 3, 6])
    v2 = oracle.sgmv(np.zeros((6, 8)), x, [A[i][None] for i in range(3)], seg)
    y2 = oracle.sgmv(np.zeros((6, 32)), v2, [B[i][None] for i in range(3)], seg)
    assert np.allclose(y2, ref, rtol=1e-5, atol=1e-4)


def test_grouped_pack_roundtrip():
    torch.manual_seed(11)
    unc, q, s, meta = gen.gen_sparse_quant4_NT(256, 256, groupsize=128, device="cpu")
    assert s.shape == (2, 256)
    w = fmt.dequantize(q.numpy(), meta.numpy(), s.numpy())
    assert np.array_equal(w, unc.numpy())
    qs, metas, ss = gen.random_packed_deltas(2, 256, 256, groupsize=128, device="cpu", seed=4)
    lev = fmt.dense_levels(qs[1].numpy(), metas[1].numpy())
    assert ((lev.reshape(64, 4, 256) != 0).sum(axis=1) == 2).all()
    assert np.abs(lev).max() <= 7


def test_tp_chunking_matches_whole():
    torch.manual_seed(12)
    unc, q, s, meta = gen.gen_sparse_quant4_NT(512, 256, device="cpu")
    scale = s  # per-channel, natural order
    qs, scs, ms = gen.torch_weight_to_sparse_marlin(unc, scale, tp_size=2, chunk_by="column")
    for i in range(2):
        w = fmt.dequantize(qs[i].numpy(), ms[i].numpy(), scs[i].numpy())
        assert np.array_equal(w, unc.numpy()[:, i * 256:(i + 1) * 256])
    qs, scs, ms = gen.torch_weight_to_sparse_marlin(unc, scale, tp_size=2, chunk_by="row")
    for i in range(2):
        w = fmt.dequantize(qs[i].numpy(), ms[i].numpy(), scs[i].numpy())
        assert np.array_equal(w, unc.numpy()[i * 128:(i + 1) * 128])
