"""Launch policy of the sm_100a attention path: ``forward(**kwargs) -> (out, lse)``.

Same private ABI as the reference's per-arch launch modules
(src/nvidia/flash_attn/sm103/launch.py:282-311; keywords listed at
python/atrex/api/flash_attn.py:396-420), plus the three context-parallel arguments the
reference's API rejects.  The caller has already validated the
call.  This module allocates what the caller did not pass (``out``, ``lse``), asks
the native launcher how much call-local scratch the call needs, takes it from the
torch allocator (so a CUDA-graph pool owns it during capture and nothing is
retained between calls, as the reference requires:
src/nvidia/flash_attn/sm103/decode_runtime.py:829-847) and enqueues the call: directly through
the C ABI in eager mode, through the custom op ``atrex_sm100::fa_fwd`` when a tracer is compiling.
The route and the split count are resolved inside the native launcher from
graph-static sizes only.

Host cost.  A serving loop repeats one call layout (shapes, strides, scalar arguments) step after
step with fresh addresses.  Filling the 70-field parameter block and asking the launcher for its plan
is most of the Python time of a call, and both depend on the layout only, so each host thread keeps
the filled block and the planned scratch size per layout and patches the addresses into it.  Nothing
read from device memory, and no tensor identity or version counter, enters the key: lengths, page
tables and descales are re-read on the device at every launch.
"""

from __future__ import annotations

import threading

import torch

from . import runtime

# Route used when the caller does not pass one: AUTO lets the native launcher choose.  Tests set this to
# pin a kernel family, the way the reference's tests observe or force a route
# (op_test/nvidia/flash_attn/test_flash_attn_sm103.py:415-427,894-930).
DEFAULT_ROUTE = runtime.ROUTE_AUTO

_LAYOUT_CACHE_LIMIT = 256
_local = threading.local()


def _layouts() -> dict:
    cache = getattr(_local, "layouts", None)
    if cache is None:
        cache = _local.layouts = {}
    return cache


def forward(*, q, k, v, cu_seqlens_q, cu_seqlens_k, seqused_k, max_seqlen_q, max_seqlen_k, page_table,
            softmax_scale, causal, softcap, window_size_left, window_size_right, learnable_sink, out,
            return_lse, q_descale, k_descale, v_descale, num_splits, route=None, cp_world_size=1, cp_rank=0,
            cp_tot_seqused_k=None, layout_token=None):
    """``layout_token``: optional hashable value that determines every argument except tensor addresses (the
    public API passes its call signature); it then serves as the layout key instead of one computed here."""
    if route is None:
        route = DEFAULT_ROUTE
    if out is None:
        out = torch.empty(q.shape, dtype=torch.bfloat16, device=q.device)
    lse = torch.empty((q.shape[1], q.shape[0]), dtype=torch.float32, device=q.device) if return_lse else None
    window_left = -1 if window_size_left is None else int(window_size_left)
    window_right = -1 if window_size_right is None else int(window_size_right)
    status = runtime.device_status(q.device)
    args = (q, k, v, out, lse, cu_seqlens_q, cu_seqlens_k, seqused_k, page_table, q_descale, k_descale,
            v_descale, learnable_sink, status, int(max_seqlen_q), int(max_seqlen_k), float(softmax_scale),
            float(softcap), bool(causal), window_left, window_right, int(num_splits), int(route),
            int(cp_world_size), int(cp_rank), cp_tot_seqused_k)
    key = (layout_token, route) if layout_token is not None else runtime.layout_key(*args)
    layouts = _layouts()
    entry = layouts.get(key)
    if entry is None:
        params = runtime.build_params(*args)
        entry = (params, runtime.plan(params).workspace_bytes)
        if len(layouts) >= _LAYOUT_CACHE_LIMIT:
            layouts.clear()
        layouts[key] = entry
    else:
        runtime.set_pointers(entry[0], *args[:14], args[25])
    params, workspace_bytes = entry
    workspace = torch.empty(workspace_bytes, dtype=torch.uint8, device=q.device) if workspace_bytes else None
    if torch.compiler.is_compiling():
        # under a tracer the call must be an operator the tracer can see
        runtime.fa_fwd(q, k, v, out, lse, workspace, *args[5:])
    else:
        runtime.launch_params(params, workspace, q.device)
    return out, lse
