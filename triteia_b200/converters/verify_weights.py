"""Checks of a converted checkpoint against a reference conversion of the same model — the
counterpart of triteia/tools/verify_weights.py (`check_tp_group_equal` :6-42, `check_output` :45-79,
`check_output_all_modules` :82-93).

Keys are `{module}.{tp_rank}.{qweight,scales,meta}`.  `check_output` pushes one random batch through
every tensor-parallel chunk of a module (the indexed delta matmul path's single-delta operator,
`matmul_4bit_2_4`) and compares the reassembled result with the same batch through the reference's
single chunk: chunks of a column-split module (fused qkv / gate_up) are concatenated along the
output features, chunks of a row-split module (o_proj / down_proj) see their slice of the input
features and are summed.
"""
import torch

from ..configs.models.llama import row_chunking_modules
from ..ops import matmul_4bit_2_4


def split_key(key):
    """`a.b.c.3.qweight` -> (`a.b.c`, 3, `qweight`)."""
    parts = key.split(".")
    return ".".join(parts[:-2]), int(parts[-2]), parts[-1]


def modules_of(weights):
    return sorted({split_key(k)[0] for k in weights if k.split(".")[-1] in ("qweight", "scales", "meta")})


def check_tp_group_equal(weights):
    """Every component of a module must exist once per tensor-parallel rank; returns the list of
    (module, component, rank_a, rank_b) whose tensors are identical (a sign of a chunking mistake)."""
    same = []
    for module in modules_of(weights):
        ranks = sorted({split_key(k)[1] for k in weights if split_key(k)[0] == module})
        for comp in ("qweight", "scales", "meta"):
            have = [r for r in ranks if f"{module}.{r}.{comp}" in weights]
            assert have == list(range(len(ranks))), f"module {module}: component {comp} present for ranks {have}"
            for a, b in zip(have, have[1:]):
                ta, tb = weights[f"{module}.{a}.{comp}"], weights[f"{module}.{b}.{comp}"]
                if ta.shape == tb.shape and torch.equal(ta, tb):
                    same.append((module, comp, a, b))
    return same


@torch.no_grad()
def check_output(weights, reference_weights, module_name, nr=128, generator=None):
    """max |reference - reassembled| / mean |reference| of one random batch of `nr` rows (the metric of
    the reference's check).  `reference_weights` holds the module converted with tp_size 1."""
    rq = reference_weights[f"{module_name}.0.qweight"]
    rm = reference_weights[f"{module_name}.0.meta"]
    rs = reference_weights[f"{module_name}.0.scales"]
    k = 32 * rq.shape[0]
    x = torch.randn((nr, k), dtype=torch.float16, device=rq.device, generator=generator)
    ref = matmul_4bit_2_4(rq, x, rm, rs)
    ranks = sorted({split_key(key)[1] for key in weights if split_key(key)[0] == module_name})
    by_rows = any(module_name.endswith(m) for m in row_chunking_modules)
    outs, at = [], 0
    for r in ranks:
        q, m, s = (weights[f"{module_name}.{r}.{c}"] for c in ("qweight", "meta", "scales"))
        if by_rows:
            kr = 32 * q.shape[0]
            outs.append(matmul_4bit_2_4(q, x[:, at:at + kr].contiguous(), m, s).float())
            at += kr
        else:
            outs.append(matmul_4bit_2_4(q, x, m, s))
    got = torch.stack(outs).sum(0) if by_rows else torch.cat(outs, dim=1)
    return float((ref.float() - got.float()).abs().max() / ref.float().abs().mean())


def check_output_all_modules(weights, reference_weights, nr=128):
    """{module: metric} for every packed module of the checkpoint."""
    return {m: check_output(weights, reference_weights, m, nr=nr) for m in modules_of(weights)}
