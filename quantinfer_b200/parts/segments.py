"""Long entries of a step cut into segments, for recurrences that are linear in their state.

A recurrence S_t = a_t S_(t-1) + b_t over an entry of many tokens runs as three launches: every segment as an entry
of its own from zeros (its own contribution to its end state), a chain over each entry's segments in order (which
also moves the request's state to the entry's end), and every segment again from the state it starts with, now with
outputs. The lists below are made once a step, on the host, and shared by the step's layers through `batch.extra`.
"""

from __future__ import annotations

import torch

from .. import kernels

SEGMENT = 64          # tokens a segment of a long entry, where nothing better is known (`segment_length` picks one a step)
SEGMENT_FROM = 192    # entries shorter than this run in one piece


def entry_segments(batch, segment: int = SEGMENT, segment_from: int = SEGMENT_FROM):
    """None when no entry of the step is long, or when the step may be replayed from a CUDA graph (it holds single
    tokens and has no host-side lists). Else (first rows of the segments [segments + 1], first segments of the entries
    [entries + 1], zeros [segments], ones [segments], scratch rows 0 .. segments - 1, most segments an entry), all but
    the last on the device."""
    if batch.extra.get("graph") or batch.max_q_len < segment_from:
        return None
    key = ("segments", segment, segment_from)
    if key not in batch.extra:
        starts, entry_seg, longest = [], [0], 0
        q = batch.h_q_start
        for a, b in zip(q[:-1], q[1:]):
            cuts = list(range(a, b, segment)) if b - a >= segment_from else [a]
            starts += cuts
            entry_seg.append(len(starts))
            longest = max(longest, len(cuts))
        n_seg = len(starts)
        host = torch.tensor(starts + [q[-1]] + entry_seg + [0] * n_seg + [1] * n_seg + list(range(n_seg)), dtype=torch.int32)
        dev = host.to(batch.q_start.device, non_blocking=True)
        o = [n_seg + 1, n_seg + 1 + len(entry_seg)]
        batch.extra[key] = (dev[:o[0]], dev[o[0]:o[1]], dev[o[1]:o[1] + n_seg], dev[o[1] + n_seg:o[1] + 2 * n_seg],
                            dev[o[1] + 2 * n_seg:], longest)
    return batch.extra[key]


def segment_length(batch, blocks_a_segment: int, blocks_at_a_time: int, segment_from: int = SEGMENT_FROM) -> int:
    """Tokens a segment for the matrix-state scan of this step: the launch has `blocks_a_segment` blocks for every segment
    and the device holds `blocks_at_a_time` of them, so a launch lasts (waves) x (a segment's tokens, plus the few tokens'
    worth that loading and storing a state costs); twice that for the two passes, plus the chain's walk over the
    longest entry's segments. The cheapest multiple of 8 between 32 and 256 by that count."""
    if blocks_at_a_time <= 0:
        return SEGMENT
    key = ("segment_length", blocks_a_segment, blocks_at_a_time, segment_from)
    if key not in batch.extra:
        q = batch.h_q_start
        lens = [b - a for a, b in zip(q[:-1], q[1:])]
        best = None
        for length in range(32, 257, 8):
            segs = [-(-n // length) if n >= segment_from else 1 for n in lens]
            waves = -(-sum(segs) * blocks_a_segment // blocks_at_a_time)
            cost = 2 * waves * (length + 6) + 0.5 * max(segs)
            if best is None or cost < best[0]:
                best = (cost, length)
        batch.extra[key] = best[1]
    return batch.extra[key]


def matrix_state_scan(mode: str, r, k, v, state, o, batch, heads: int, dk: int, dv: int, **operands) -> None:
    """`kernels.matrix_state_scan` over the step's entries: in one launch, or, when an entry is long, segment by
    segment as the module's head describes. state [slots, heads, dv, dk]; o float32 [n, heads dv]."""
    if batch.extra.get("graph") or batch.max_q_len < SEGMENT_FROM:
        seg = None
    else:
        col_blocks = -(-dv // kernels.MATRIX_STATE_COLUMNS)
        seg = entry_segments(batch, segment_length(batch, heads * col_blocks, kernels.matrix_state_scan_blocks(mode, dk, r.dtype)))
    if seg is None:
        return kernels.matrix_state_scan(mode, r, k, v, state, o, batch.q_start, batch.start_pos, batch.slot_ids, heads, dk, dv, **operands)
    seg_q_start, entry_seg, zeros, ones, rows, _ = seg
    own = torch.empty((rows.numel(), heads, dv, dk), dtype=torch.float32, device=o.device)
    decay = torch.empty((rows.numel(), heads, dk), dtype=torch.float32, device=o.device)
    kernels.matrix_state_scan(mode, r, k, v, own, None, seg_q_start, zeros, rows, heads, dk, dv, decay_out=decay, **operands)
    kernels.matrix_state_chain(own, decay, state, entry_seg, batch.start_pos, batch.slot_ids)
    kernels.matrix_state_scan(mode, r, k, v, own, o, seg_q_start, ones, rows, heads, dk, dv, write_state=False, **operands)
