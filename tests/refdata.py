"""Seeded synthetic inputs for the parity tests and the bench (test infrastructure).

Two generators:
* a counter-based hash (splitmix64 finaliser) -> uniform / normal arrays that depend only on
  (seed, index), so fixtures store outputs and every machine regenerates identical inputs;
* `kaiming_uniform`, a numpy restatement of how the reference draws layer weights:
  std::mt19937(0xC0FFEE) feeding std::uniform_real_distribution<float>(-b, b) with
  b = sqrt(1 / fan_in) (nn/Linear.cpp:21-29, nn/Conv2dModule.cpp:88-97). libstdc++ draws one
  32-bit word per float: canonical = float(word) / 2^32 (clamped below 1), value =
  canonical * (b - a) + a. tests/test_oracle_pins.py pins it against the reference itself.
"""
import numpy as np

MNIST_MEAN, MNIST_STD = 0.1307, 0.3081  # data/MnistLoader.cpp:26-28


def _mix(seed, n, stream=0):
    with np.errstate(over="ignore"):
        x = np.arange(n, dtype=np.uint64) + np.uint64((seed * 0x9E3779B97F4A7C15 + stream * 0xD1B54A32D192ED03) % 2**64)
        x = (x + np.uint64(0x9E3779B97F4A7C15))
        x ^= x >> np.uint64(30)
        x *= np.uint64(0xBF58476D1CE4E5B9)
        x ^= x >> np.uint64(27)
        x *= np.uint64(0x94D049BB133111EB)
        x ^= x >> np.uint64(31)
    return x


def uniform(seed, shape, lo=-1.0, hi=1.0):
    """i.i.d. uniform [lo, hi) as float32."""
    n = int(np.prod(shape))
    u = (_mix(seed, n) >> np.uint64(40)).astype(np.float64) / float(1 << 24)  # 24-bit fraction, < 1
    return (lo + (hi - lo) * u).astype(np.float32).reshape(shape)


def normal(seed, shape):
    """i.i.d. N(0, 1) as float32 (Box-Muller on two hashed uniforms)."""
    n = int(np.prod(shape))
    u1 = ((_mix(seed, n, 1) >> np.uint64(11)).astype(np.float64) + 1.0) / float(1 << 53)
    u2 = (_mix(seed, n, 2) >> np.uint64(11)).astype(np.float64) / float(1 << 53)
    z = np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)
    return z.astype(np.float32).reshape(shape)


def labels(seed, n, classes=10):
    return (_mix(seed, n, 3) % np.uint64(classes)).astype(np.int64)


def mnist_like(seed, shape):
    """uniform [0,1) pixels with the MNIST normalisation the reference's loader applies."""
    px = uniform(seed, shape, 0.0, 1.0)
    return ((px - np.float32(MNIST_MEAN)) / np.float32(MNIST_STD)).astype(np.float32)


def kaiming_uniform(shape, fan_in, seed=0xC0FFEE):
    n = int(np.prod(shape))
    rs = np.random.RandomState(seed)
    words = rs.randint(0, 2**32, size=n, dtype=np.uint64).astype(np.uint32)
    c = (words.astype(np.float32) / np.float32(4294967296.0)).astype(np.float32)
    c = np.where(c >= np.float32(1.0), np.nextafter(np.float32(1.0), np.float32(0.0)), c).astype(np.float32)
    bound = np.sqrt(np.float32(1.0) / np.float32(fan_in)).astype(np.float32)
    return (c * (bound - (-bound)) + (-bound)).astype(np.float32).reshape(shape)


def linear_weight(in_f, out_f):
    return kaiming_uniform((out_f, in_f), in_f)


def conv_weight(cin, cout, k):
    return kaiming_uniform((cout, cin, k, k), cin * k * k)


def to_bf16_bits(a):
    """float32 -> bf16 bit patterns (uint16), round to nearest even."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return r.astype(np.uint16)


def from_bf16_bits(b):
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


# Fill patterns of the reference's own kernel tests.
def gemm_test_patterns():
    """(name, A, B) as in cuda/kernels/gemm_{naive,tiled_16x16,optimized}_test.cpp."""
    f = np.float32
    cases = []
    cases.append(("2x2", np.array([[1, 2], [3, 4]], f), np.array([[5, 6], [7, 8]], f)))
    cases.append(("identity4", np.arange(1, 17, dtype=f).reshape(4, 4), np.eye(4, dtype=f)))
    a = np.arange(1, 16, dtype=f).reshape(3, 5)
    b = (f(0.1) * np.arange(1, 11, dtype=f)).reshape(5, 2)
    cases.append(("3x5x2", a, b))
    M, K, N = 17, 19, 23
    a = (f(0.01) * np.arange(1, M * K + 1, dtype=f)).reshape(M, K)
    b = (f(0.02) * ((np.arange(K * N) % 7) + 1).astype(f)).reshape(K, N)
    cases.append(("17x19x23", a, b))
    for n in (16, 32):
        a = (f(0.1) * np.arange(1, n * n + 1, dtype=f)).reshape(n, n)
        b = (f(0.05) * ((np.arange(n * n) % 7) + 1).astype(f)).reshape(n, n)
        cases.append((f"sq{n}", a, b))
    n = 64
    a = (f(0.01) * np.arange(1, n * n + 1, dtype=f)).reshape(n, n)
    b = (f(0.02) * ((np.arange(n * n) % 11) + 1).astype(f)).reshape(n, n)
    cases.append(("sq64", a, b))
    cases.append(("zeros4", np.zeros((4, 4), f), np.ones((4, 4), f)))
    return cases
