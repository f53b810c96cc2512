"""numpy re-statement of the input generator the reference's kernel tests use
(tests/kernels/test_rmsnorm.cpp:19-29 and its copies): std::mt19937(seed) feeding
std::uniform_real_distribution<float>(-scale, scale), each value rounded to bf16.
libstdc++ draws one 32-bit word per value: u = float(word) / 2^32 (clamped below 1), then
u * (b - a) + a in float.  Pinned against the compiled reference in test_oracle_golden.py."""
import numpy as np


def f32_to_bf16(f: np.ndarray) -> np.ndarray:
    u = f.astype(np.float32).view(np.uint32)
    nan = (u & 0x7fffffff) > 0x7f800000
    r = ((u + (0x7fff + ((u >> 16) & 1))) >> 16).astype(np.uint16)
    r[nan] = 0x7fff
    return r


def make_bf16_random(count: int, scale: float, seed: int) -> np.ndarray:
    bg = np.random.MT19937()
    bg._legacy_seeding(seed)
    words = bg.random_raw(count).astype(np.uint32)
    u = words.astype(np.float32) / np.float32(4294967296.0)
    u = np.where(u >= np.float32(1.0), np.nextafter(np.float32(1.0), np.float32(0.0)), u).astype(np.float32)
    a, b = np.float32(-scale), np.float32(scale)
    v = (u * np.float32(b - a)).astype(np.float32) + a
    return f32_to_bf16(v.astype(np.float32))
