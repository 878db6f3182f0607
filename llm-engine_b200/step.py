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
