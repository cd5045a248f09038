"""Seeded synthetic GGUF-layout tensors for tests and benchmarks.

No model files are available, so weights are synthetic blocks with the recipes the benchmark configurations
name: random code bytes and a small positive f16 block scale written at the type's scale offset. This is the
reference's own recipe for types no model holds (tests/gpu/test_q8_gpu.hip:181-193, tests/test_cpu_q8.c:34-56),
with the scale distribution |N(0,1)| * sigma.
"""
import numpy as np

# type id -> (values, bytes)
BLOCK = {2: (32, 18), 8: (32, 34), 10: (256, 84), 12: (256, 144), 16: (256, 66), 17: (256, 74), 18: (256, 98),
         19: (256, 50), 22: (256, 82), 29: (256, 56), 39: (32, 17), 40: (64, 36),
         7: (32, 24), 11: (256, 110), 13: (256, 176), 14: (256, 210), 20: (32, 18), 23: (256, 136), 42: (64, 18),
         43: (32, 33), 0: (1, 4), 30: (1, 2)}
TYPE_ID = {"Q4_0": 2, "Q8_0": 8, "Q2_K": 10, "Q4_K": 12, "IQ2_XXS": 16, "IQ2_XS": 17, "IQ3_XXS": 18, "IQ1_S": 19,
           "IQ2_S": 22, "IQ1_M": 29, "MXFP4": 39, "NVFP4": 40, "Q5_1": 7, "Q3_K": 11, "Q5_K": 13, "Q6_K": 14,
           "IQ4_NL": 20, "IQ4_XS": 23, "Q2_0": 42, "MXFP8": 43, "F32": 0, "BF16": 30}
SEED = 1017


def tensor_bytes(type_id, rows, cols):
    values, nbytes = BLOCK[type_id]
    assert cols % values == 0, (type_id, cols)
    return rows * (cols // values) * nbytes


def _f16_bits(rng, n, sigma):
    d = (np.abs(rng.standard_normal(n)) * sigma).astype(np.float16)
    d = np.maximum(d, np.float16(6e-5))  # keep scales normal and non-zero
    return d.view(np.uint16)


def random_blocks(type_id, n_blocks, rng, sigma=0.01):
    """n_blocks blocks of `type_id` as a uint8 array [n_blocks, block_bytes]."""
    values, nbytes = BLOCK[type_id]
    if type_id in (0, 30):  # unquantized: a "block" is one value, N(0, 1) * sigma
        v = (rng.standard_normal(n_blocks) * sigma).astype(np.float32)
        if type_id == 0:
            return v.view(np.uint8).reshape(n_blocks, 4).copy()
        return (v.view(np.uint32) >> 16).astype(np.uint16).view(np.uint8).reshape(n_blocks, 2).copy()
    raw = rng.integers(0, 256, size=(n_blocks, nbytes), dtype=np.uint8)
    if type_id == 43:  # MXFP8: E8M0 exponent byte with bias 127; E4M3 codes without the two NaN codes
        raw[:, 0] = rng.integers(117, 124, size=n_blocks, dtype=np.uint8)
        codes = raw[:, 1:]
        codes[(codes & 0x7F) == 0x7F] = 0x38
        return raw
    if type_id == 39:  # MXFP4: E8M0 exponent byte, 2^-10 .. 2^-4 with bias 127
        raw[:, 0] = rng.integers(117, 124, size=n_blocks, dtype=np.uint8)
        return raw
    if type_id == 40:  # NVFP4: four UE4M3 scale bytes, kept finite and positive
        raw[:, 0:4] = rng.integers(0x20, 0x48, size=(n_blocks, 4), dtype=np.uint8)
        return raw
    d = _f16_bits(rng, n_blocks, sigma)
    if type_id == 29:  # IQ1_M: the f16 scale lives in the top nibbles of the four 16-bit scale words
        for k in range(4):
            hi = raw[:, 48 + 2 * k + 1]
            raw[:, 48 + 2 * k + 1] = (hi & 0x0F) | ((((d >> (4 * k)) & 0x0F).astype(np.uint8)) << 4)
        return raw
    if type_id == 10:  # Q2_K: d and dmin after the scales and codes
        m = _f16_bits(rng, n_blocks, sigma)
        raw[:, 80] = d & 0xFF
        raw[:, 81] = d >> 8
        raw[:, 82] = m & 0xFF
        raw[:, 83] = m >> 8
        return raw
    if type_id in (11, 14):  # Q3_K, Q6_K: d is the block's last two bytes
        raw[:, nbytes - 2] = d & 0xFF
        raw[:, nbytes - 1] = d >> 8
        return raw
    raw[:, 0] = d & 0xFF
    raw[:, 1] = d >> 8
    if type_id in (12, 13, 7):  # Q4_K, Q5_K: dmin right after d; Q5_1: its minimum
        m = _f16_bits(rng, n_blocks, sigma)
        raw[:, 2] = m & 0xFF
        raw[:, 3] = m >> 8
    return raw


def random_tensor(type_id, rows, cols, rng, sigma=0.01):
    """A row-major rows x cols tensor of `type_id` as a flat uint8 array."""
    values, _ = BLOCK[type_id]
    return random_blocks(type_id, rows * (cols // values), rng, sigma).reshape(-1)


def rng_for(*key):
    return np.random.default_rng([SEED, *[int(k) for k in key]])
