"""Rotary position embedding, in place; same functions as
triteia/python/capi/rotary_embedding.py:5-38."""
from .. import triteia_cuda


def rotary_embedding(positions, query, key, head_size, cos_sin_cache, is_neox) -> None:
    triteia_cuda.rotary_embedding(positions, query, key, head_size, cos_sin_cache, is_neox)


def batched_rotary_embedding(positions, query, key, head_size, cos_sin_cache, is_neox, rot_dim,
                             cos_sin_cache_offsets) -> None:
    triteia_cuda.batched_rotary_embedding(positions, query, key, head_size, cos_sin_cache, is_neox, rot_dim,
                                          cos_sin_cache_offsets)
