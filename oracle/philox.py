"""Philox4x32-10 and bf16 stochastic rounding, NumPy restatement (test oracle).

Follows the generator the reference reaches through ``tl.randint``
(triton/language/random.py: philox_impl, randint4x — the reference's call
sites are shared_ffi/sr_triton.py:11 and :163) and the rounding rule of
shared_ffi/sr_triton.py:10-16.
"""
import numpy as np

PHILOX_KEY_A = 0x9E3779B9
PHILOX_KEY_B = 0xBB67AE85
PHILOX_ROUND_A = 0xD2511F53
PHILOX_ROUND_B = 0xCD9E8D57
_M32 = np.uint64(0xFFFFFFFF)


def philox4x32(c0, c1, c2, c3, k0, k1, rounds=10):
    """Counter (c0..c3) and key (k0,k1) are uint32 arrays/scalars; returns 4 uint32 arrays."""
    c0 = np.asarray(c0, dtype=np.uint64) & _M32
    c1 = np.asarray(c1, dtype=np.uint64) & _M32
    c2 = np.asarray(c2, dtype=np.uint64) & _M32
    c3 = np.asarray(c3, dtype=np.uint64) & _M32
    c0, c1, c2, c3 = np.broadcast_arrays(c0, c1, c2, c3)
    k0 = np.uint64(int(k0) & 0xFFFFFFFF)
    k1 = np.uint64(int(k1) & 0xFFFFFFFF)
    A = np.uint64(PHILOX_ROUND_A)
    B = np.uint64(PHILOX_ROUND_B)
    for _ in range(rounds):
        pa = A * c0          # 64-bit product of two 32-bit values
        pb = B * c2
        n0 = (pb >> np.uint64(32)) ^ c1 ^ k0
        n2 = (pa >> np.uint64(32)) ^ c3 ^ k1
        n1 = pb & _M32
        n3 = pa & _M32
        c0, c1, c2, c3 = n0, n1, n2, n3
        k0 = (k0 + np.uint64(PHILOX_KEY_A)) & _M32
        k1 = (k1 + np.uint64(PHILOX_KEY_B)) & _M32
    return (c0.astype(np.uint32), c1.astype(np.uint32), c2.astype(np.uint32), c3.astype(np.uint32))


def randint_ref(seed, offsets):
    """``tl.randint(seed, offsets)`` for int32 offsets: counter (offset,0,0,0), key (seed_lo, seed_hi), word 0."""
    seed = int(seed) & 0xFFFFFFFFFFFFFFFF
    off = np.asarray(offsets).astype(np.int64).astype(np.uint64) & _M32
    w0, _, _, _ = philox4x32(off, 0, 0, 0, seed & 0xFFFFFFFF, seed >> 32)
    return w0


def rand16_reference(seed, flat_offsets):
    """16 random bits per element, reference stream (sr_triton.py:11: ``randint & 65535``)."""
    return (randint_ref(seed, flat_offsets) & np.uint32(0xFFFF)).astype(np.uint32)


def rand16_packed(seed, step, rows, cols):
    """16 random bits per element, packed stream: one Philox call feeds eight slots.

    key = (seed, step), counter = (row, col >> 3, 0, 0); slot ``col`` takes the
    16-bit half ``col & 1`` of word ``(col & 7) >> 1``.  ``rows`` is the GLOBAL
    label index so the bits do not depend on how labels are sharded.
    """
    rows = np.asarray(rows, dtype=np.int64)
    cols = np.asarray(cols, dtype=np.int64)
    rows, cols = np.broadcast_arrays(rows, cols)
    w = philox4x32(rows.astype(np.uint64), (cols >> 3).astype(np.uint64), 0, 0,
                   int(seed) & 0xFFFFFFFF, int(step) & 0xFFFFFFFF)
    word = np.choose(((cols & 7) >> 1).astype(np.int64), w)
    return ((word >> (16 * (cols & 1)).astype(np.uint32)) & np.uint32(0xFFFF)).astype(np.uint32)


def f32_bits(x):
    return np.ascontiguousarray(np.asarray(x, dtype=np.float32)).view(np.uint32)


def sr_bf16_bits(w32, r16):
    """Stochastic rounding fp32 -> bf16 (returned as uint16 bit patterns).

    sr_triton.py:10-16: add 16 random bits to the fp32 bit pattern as an
    integer, clear the low half, keep the high half.  On sign-magnitude floats
    this rounds away from zero with probability low16/65536.
    """
    bits = f32_bits(w32).astype(np.uint64)
    out = (bits + np.asarray(r16, dtype=np.uint64)) & np.uint64(0xFFFF0000)
    return ((out & _M32) >> np.uint64(16)).astype(np.uint16)


def bf16_bits_to_f32(b16):
    return (np.asarray(b16, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def rn_bf16_bits(x32):
    """Round-to-nearest-even fp32 -> bf16 bit patterns (finite inputs)."""
    bits = f32_bits(x32).astype(np.uint64)
    lsb = (bits >> np.uint64(16)) & np.uint64(1)
    out = (bits + np.uint64(0x7FFF) + lsb) >> np.uint64(16)
    return (out & np.uint64(0xFFFF)).astype(np.uint16)
