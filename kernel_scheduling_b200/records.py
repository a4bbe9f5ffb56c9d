"""Binary layouts shared by the host code and the CUDA library.

Launch record (48 bytes, little endian). It carries the fields of one row of the agent's timing log
(reference: scheduler/agent.cpp:500-508 ``TimingResult`` and the 17-column writer at :692-705) that the
trace -> interference-table path needs, with the kernel name already replaced by a dictionary id:

    offset  0  u32  name_id       id of the canonical kernel name (see ``names.function_base``)
    offset  4  u32  grid[3]       grid x, y, z
    offset 16  u32  block[3]      block x, y, z
    offset 28  u32  smem_word     bits 0..22 dynamic shared memory in bytes, bit 23 solo flag, bits 24..31 tenant
    offset 32  u64  start_ns      CLOCK_MONOTONIC ns when the launch was queued (agent.cpp:960-963)
    offset 40  u64  end_ns        CLOCK_MONOTONIC ns when the completion callback ran (agent.cpp:139-146)

The tenant is the process / SCHED_MODEL the launch came from (scheduler_daemon.cpp:210-213 puts the model
in the key); the solo flag marks launches of a one-kernel-at-a-time run (pairprof_daemon.cpp:46,190).
"""
from __future__ import annotations

import numpy as np

RECORD_DTYPE = np.dtype(
    [
        ("name_id", "<u4"),
        ("grid", "<u4", (3,)),
        ("block", "<u4", (3,)),
        ("smem_word", "<u4"),
        ("start_ns", "<u8"),
        ("end_ns", "<u8"),
    ]
)
assert RECORD_DTYPE.itemsize == 48

SMEM_MASK = 0x007FFFFF
SOLO_BIT = 1 << 23
TENANT_SHIFT = 24

# key modes (which launch fields make up the kernel key)
KEY_SHAPE = 0  # tenant, name, block, grid, smem        (a SHAPE row of scheduler_daemon.cpp:196-197)
KEY_TYPE = 1   # tenant, name, block                     (a TYPE row: grid "*")

# One row of the pair table as the library returns it (128 bytes).
PAIR_ROW_DTYPE = np.dtype(
    [
        ("key_a", "<u8"),
        ("key_b", "<u8"),
        ("count", "<u8"),
        ("flags", "<u8"),  # bit 0: side a has a solo baseline, bit 1: side b has one
        ("sum_a", "<f8"),
        ("mean_a", "<f8"),
        ("min_a", "<f8"),
        ("max_a", "<f8"),
        ("median_a", "<f8"),
        ("sum_b", "<f8"),
        ("mean_b", "<f8"),
        ("min_b", "<f8"),
        ("max_b", "<f8"),
        ("median_b", "<f8"),
        ("efficiency", "<f8"),  # median over occurrences of (solo_a + solo_b) / (max(end) - min(start))
        ("span_sum_ns", "<u8"),  # sum over occurrences of max(end) - min(start)
    ]
)
assert PAIR_ROW_DTYPE.itemsize == 128

# One row of the per-key table (72 bytes).
KEY_ROW_DTYPE = np.dtype(
    [
        ("key", "<u8"),
        ("name_id", "<u4"),
        ("grid", "<u4", (3,)),
        ("block", "<u4", (3,)),
        ("smem", "<u4"),
        ("tenant", "<u4"),
        ("reserved", "<u4"),
        ("launches", "<u8"),
        ("solo_launches", "<u8"),
        ("solo_ns", "<f8"),  # exact median of end_ns - start_ns over the key's solo launches; NaN if none
    ]
)
assert KEY_ROW_DTYPE.itemsize == 72


def pack_records(name_id, grid, block, smem, tenant, solo, start_ns, end_ns) -> np.ndarray:
    """Builds a record array from column arrays (all of one length)."""
    n = len(name_id)
    rec = np.zeros(n, dtype=RECORD_DTYPE)
    rec["name_id"] = name_id
    rec["grid"] = np.asarray(grid, dtype=np.uint32).reshape(n, 3)
    rec["block"] = np.asarray(block, dtype=np.uint32).reshape(n, 3)
    smem = np.asarray(smem, dtype=np.uint64)
    tenant = np.asarray(tenant, dtype=np.uint64)
    if n and (smem.max() > SMEM_MASK or tenant.max() > 255):
        raise ValueError("dynamic shared memory must be < 2**23 bytes and tenant < 256")
    solo = np.asarray(solo, dtype=bool)
    rec["smem_word"] = (smem | (solo.astype(np.uint64) << np.uint64(23)) | (tenant << np.uint64(TENANT_SHIFT))).astype(np.uint32)
    rec["start_ns"] = start_ns
    rec["end_ns"] = end_ns
    return rec


def unpack_smem_word(word: np.ndarray):
    """-> (smem bytes, solo flag, tenant)"""
    word = np.asarray(word, dtype=np.uint32)
    return word & np.uint32(SMEM_MASK), (word & np.uint32(SOLO_BIT)) != 0, word >> np.uint32(TENANT_SHIFT)
