"""CPU restatement of the KV-cache write step (TEST INFRASTRUCTURE: only tests/, smoke() and bench.py's CPU
baseline may import this; the product path never does).

PARITY UNPINNED against the reference: alibaba/atrex-kernels has no cache writer -- its tests fill the paged
pools by indexing (op_test/utils/flash_attn_contract.py:40-51).  The semantics restated here are the serving
engines' published reshape-and-cache step: token ``t`` is stored at ``slot_mapping[t] = page * page_size + row``
(negative slots are padding and are skipped), an FP8 cache stores ``e4m3(x / scale[head])`` rounded to nearest
even and saturated at +-448.  It is anchored to the reference in two ways: the E4M3 rounding is the one the
attention oracle uses and is pinned against torch's conversion (tests/test_oracle.py), and tests/ check that
attention over a cache written this way equals the pinned attention oracle over the same rows laid out by
indexing, the way the reference's tests build their caches.
"""

from __future__ import annotations

import numpy as np

from . import fa_oracle


def write_kv_cache(key, value, key_cache, value_cache, slot_mapping, k_scale=None, v_scale=None, fp8=False):
    """``key`` / ``value`` float32 [T, H, D] (already BF16-representable); caches float32 [P, page, H, D] are
    updated in place and hold the VALUES the device cache would decode to (E4M3-rounded quotients for fp8)."""
    page = key_cache.shape[1]
    heads = key.shape[1]

    def per_head(scale):
        if scale is None:
            return np.ones(heads, dtype=np.float32)
        scale = np.asarray(scale, dtype=np.float32).reshape(-1)
        return np.broadcast_to(scale, (heads,)) if scale.size == 1 else scale

    ks, vs = per_head(k_scale), per_head(v_scale)
    for t, slot in enumerate(np.asarray(slot_mapping).tolist()):
        if slot < 0:
            continue
        p, r = divmod(slot, page)
        if fp8:
            with np.errstate(over="ignore"):   # a quotient beyond FP32 saturates like any other large value
                key_cache[p, r] = fa_oracle.e4m3_round((key[t] / ks[:, None]).astype(np.float32))
                value_cache[p, r] = fa_oracle.e4m3_round((value[t] / vs[:, None]).astype(np.float32))
        else:
            key_cache[p, r] = key[t]
            value_cache[p, r] = value[t]


def kv_scales(key, value, slot_mapping):
    """Per-head E4M3 scales: max |x| over the non-padding tokens / 448 in float32; 1.0 where that maximum is zero
    or not finite."""
    keep = np.asarray(slot_mapping) >= 0

    def one(x):
        x = np.asarray(x, dtype=np.float32)[keep]
        heads = x.shape[1]
        out = np.ones(heads, dtype=np.float32)
        if x.shape[0] == 0:
            return out
        amax = np.abs(x).max(axis=(0, 2))
        ok = np.isfinite(amax) & (amax > 0)
        out[ok] = (amax[ok] / np.float32(448.0)).astype(np.float32)
        return out

    return one(key), one(value)


def algorithmic_bytes(tokens_written, num_kv_heads, head_dim, fp8):
    """K and V rows read as BF16 and written once, plus the slot ids."""
    row = num_kv_heads * head_dim
    return tokens_written * (2 * row * 2 + 2 * row * (1 if fp8 else 2) + 8)
