"""What the mixers with a recurrent state share: how a step's long portions are cut into chunks for their scans."""

from __future__ import annotations

from .. import kernels as K


def scan_chunks(ctx):
    """The step's :class:`~litinfer_b200.kernels.ScanChunks`, made once per step from its host-side metadata and shared
    by every layer, or None: a step of single tokens or short portions, whose sequences each run in one piece (such a
    step reads its metadata on the device alone and can be replayed from a captured graph)."""
    if ctx.max_q_len < K.ScanChunks.FROM or not ctx.host_q_start:
        return None
    plan = ctx.scratch.get("scan_chunks")
    if plan is None:
        plan = K.ScanChunks(ctx.host_q_start, ctx.host_state_slots, ctx.q_start.device)
        ctx.scratch["scan_chunks"] = plan
    return plan
