"""Step-index packing: mirror of CudaModel::upload_step_indices
(llm-engine src/model/cuda/cuda_model.cu:453-473) over pkv_step_pack."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _lib


@dataclass
class StepIndices:
    slots: np.ndarray         # [N] int32: pool row each packed token's K/V is written to
    token_seq: np.ndarray     # [N] int32: step-local sequence index
    token_pos: np.ndarray     # [N] int32: absolute position
    block_tables: np.ndarray  # concatenated tables of the distinct sequences
    table_offset: np.ndarray  # [S] int32: start of each sequence's table

    @property
    def n_tokens(self) -> int:
        return int(self.token_pos.shape[0])

    @property
    def n_seqs(self) -> int:
        return int(self.table_offset.shape[0])


def pack_step(tok_tables, tok_pos, block_size: int, tok_keys=None) -> StepIndices:
    """tok_tables[i]: int32 array, block table of packed token i's sequence (tokens of one
    sequence pass the same array); tok_pos[i]: its absolute position; tok_keys[i]: sequence
    identity (defaults to id() of the table object, the analogue of the reference's
    Sequence pointer)."""
    n = len(tok_pos)
    L = _lib.lib()
    tables = [np.ascontiguousarray(t, dtype=np.int32) for t in tok_tables]
    if tok_keys is None:
        tok_keys = [id(t) for t in tok_tables]
    keys = np.ascontiguousarray(tok_keys, dtype=np.uint64)
    pos = np.ascontiguousarray(tok_pos, dtype=np.int32)
    nblk = np.ascontiguousarray([t.size for t in tables], dtype=np.int32)
    ptrs = (C.c_void_p * max(n, 1))(*[t.ctypes.data for t in tables])
    uniq = {}
    for k, t in zip(keys.tolist(), tables):
        uniq.setdefault(k, t.size)
    cap_tables = max(sum(uniq.values()), 1)
    cap_off = max(len(uniq), 1)
    slots = np.zeros(n, dtype=np.int32)
    token_seq = np.zeros(n, dtype=np.int32)
    out_tables = np.zeros(cap_tables, dtype=np.int32)
    out_off = np.zeros(cap_off, dtype=np.int32)
    n_seqs, n_table = C.c_int(0), C.c_int(0)
    st = L.pkv_step_pack(n, keys.ctypes.data, C.cast(ptrs, C.c_void_p), nblk.ctypes.data, pos.ctypes.data,
                         block_size, slots.ctypes.data, token_seq.ctypes.data, out_tables.ctypes.data,
                         cap_tables, out_off.ctypes.data, cap_off, C.byref(n_seqs), C.byref(n_table))
    _lib.check("pkv_step_pack", st)
    return StepIndices(slots, token_seq, pos, out_tables[:n_table.value].copy(), out_off[:n_seqs.value].copy())


class DeviceStepPacker:
    """Device-resident block tables plus the per-step index build of pkv_step_pack_device
    (replaces all of CudaModel::upload_step_indices, src/model/cuda/cuda_model.cu:453-491).

    The caller mirrors its sequences' tables into rows with `set_block` / `release` (queued on
    the host, sent with the next step) and calls `pack(slices)` once per step; the index arrays
    come back as device tensors, and nothing synchronises unless `check=True`."""

    def __init__(self, max_rows: int, max_blocks_per_seq: int, block_size: int, max_tokens: int,
                 max_table_entries: int, device="cuda"):
        import torch
        self.torch = torch
        self.max_rows, self.stride, self.block_size = max_rows, max_blocks_per_seq, block_size
        self.max_tokens, self.max_table = max_tokens, max_table_entries
        i32 = dict(dtype=torch.int32, device=device)
        self.seq_tables = torch.zeros((max_rows, max_blocks_per_seq), **i32)
        self.seq_nblocks = torch.zeros(max_rows, **i32)
        self.slots = torch.zeros(max_tokens, **i32)
        self.token_seq = torch.zeros(max_tokens, **i32)
        self.positions = torch.zeros(max_tokens, **i32)
        self.tables = torch.zeros(max_table_entries, **i32)
        self.table_offset = torch.zeros(4096, **i32)
        self.counts = torch.zeros(4, **i32)
        self._updates: list[tuple[int, int, int]] = []
        self._staging = torch.zeros((4096 * 2 + 1024, 3), dtype=torch.int32).pin_memory()
        self._dev_staging = torch.zeros_like(self._staging, device=device)
        self._copied = None

    def set_block(self, row: int, index: int, block_id: int) -> None:
        self._updates.append((row, index, block_id))

    def set_table(self, row: int, blocks) -> None:
        for i, b in enumerate(blocks):
            self._updates.append((row, i, int(b)))

    def release(self, row: int) -> None:
        self._updates.append((row, -1, 0))

    def pack(self, slices, check: bool = False, stream=None):
        """slices: iterable of (row, first_position, length).  Returns n_tokens (host int, the
        sum of the lengths); the device arrays are the attributes of this object."""
        torch = self.torch
        sl = np.ascontiguousarray(list(slices), dtype=np.int32).reshape(-1, 3)
        up = np.ascontiguousarray(self._updates, dtype=np.int32).reshape(-1, 3)
        self._updates = []
        n_up, n_sl = up.shape[0], sl.shape[0]
        if n_up + n_sl > self._staging.shape[0]:
            self._staging = torch.zeros((n_up + n_sl, 3), dtype=torch.int32).pin_memory()
            self._dev_staging = torch.zeros_like(self._staging, device=self.slots.device)
        if self._copied is not None:
            self._copied.synchronize()                 # the previous step's copy has left the pinned buffer
        host = self._staging.numpy()
        host[:n_up] = up
        host[n_up:n_up + n_sl] = sl
        self._dev_staging[:n_up + n_sl].copy_(self._staging[:n_up + n_sl], non_blocking=True)   # the step's one copy
        self._copied = torch.cuda.Event()
        self._copied.record()
        s = stream if stream is not None else torch.cuda.current_stream().cuda_stream
        st = _lib.lib().pkv_step_pack_device(
            self._dev_staging.data_ptr(), n_up, self._dev_staging.data_ptr() + 12 * n_up, n_sl,
            self.seq_tables.data_ptr(), self.seq_nblocks.data_ptr(), self.max_rows, self.stride, self.block_size,
            self.slots.data_ptr(), self.token_seq.data_ptr(), self.positions.data_ptr(), self.max_tokens,
            self.tables.data_ptr(), self.max_table, self.table_offset.data_ptr(), self.counts.data_ptr(), s)
        _lib.check("pkv_step_pack_device", st)
        if check:
            c = self.counts.cpu().numpy()
            if c[3] != 0:
                raise RuntimeError(f"pkv_step_pack_device: status bits {int(c[3])} (1 tables_cap, 2 tokens_cap, "
                                   f"4 position beyond table, 8 bad row)")
        return int(sl[:, 2].clip(min=0).sum()) if n_sl else 0
