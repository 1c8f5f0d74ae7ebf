"""The arithmetic of the native FP8 prefill route, restated in numpy and held against the fp64 expert on the CPU.

dr_moe_prefill_fp8 gives the tensor cores E4M3 weights as they are and a token operand made of three E4M3 terms per
entry (value, residual, residual of the residual) of x * s[kb] / c_t for gate/up (the chunk's block scale rides on the
token operand) and of act / c_t for the down projection (scales applied per chunk accumulator); fp32 accumulation, an
fp16 intermediate. This test follows those steps with exact products (float64) and shows what the scheme itself costs:
a per-row relative L2 of a few 1e-4, whatever the spread of the block scales. The kernels are compared with the same
fp64 expert in tests/test_gpu_fp8.py."""

import numpy as np

from drama_rs_b200 import synth
from oracle import moe_oracle as orc

E4M3 = synth.e4m3_values().astype(np.float64)


def split3(v: np.ndarray) -> np.ndarray:
    """Sum of three E4M3 roundings: of v, of what that left, and of what that left."""
    out = np.zeros_like(v)
    r = v.copy()
    for _ in range(3):
        q = E4M3[synth.to_e4m3(r.astype(np.float32))]
        out += q
        r = r - q
    return out


def grouped_matmul(w_codes, scales, x, fold_scale: bool) -> np.ndarray:
    """x [n, K] times the block-FP8 matrix (codes [R, K], scales [R / 128, K / 128]) transposed, the kernel's way."""
    r, k = w_codes.shape
    w = E4M3[w_codes]
    y = np.zeros((x.shape[0], r))
    rmax = np.abs(x).max(axis=1)
    for br in range(r // 128):
        rows = slice(128 * br, 128 * br + 128)
        s = scales[br].astype(np.float64)
        c = rmax * (np.abs(s).max() if fold_scale else 1.0) / 256.0
        c[c <= 1e-30] = 1.0
        acc = np.zeros((x.shape[0], 128))
        for kb in range(k // 128):
            cols = slice(128 * kb, 128 * kb + 128)
            if fold_scale:  # gate/up: one accumulator over the whole K
                acc += split3(x[:, cols] * (s[kb] / c)[:, None]) @ w[rows, cols].T
            else:  # down: one accumulator per chunk, its scale applied when it is drained
                acc += s[kb] * (split3(x[:, cols] / c[:, None]) @ w[rows, cols].T)
        y[:, rows] = acc * c[:, None]
    return y


def test_three_term_scheme_against_the_fp64_expert():
    shape = synth.MoeShape(experts=2)
    host = synth.make_fp8_experts(21, shape)
    rng = np.random.Generator(np.random.PCG64(81))
    for k in ("moe.gate_up.fp8_s", "moe.down.fp8_s"):  # block scales from 1e-6 to 1e-2
        host[k] = (host[k] * np.exp(rng.uniform(np.log(0.01), np.log(100.0), size=host[k].shape))).astype(np.float32)
    x = synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(rng.standard_normal((6, 2048), dtype=np.float32))).astype(np.float64)
    x[3] = 0.0  # an all-zero row has no normaliser of its own
    e = 1
    h = grouped_matmul(host["moe.gate_up.fp8"][e], host["moe.gate_up.fp8_s"][e], x, fold_scale=True)
    g, u = h[:, :512], h[:, 512:]
    act = (g / (1.0 + np.exp(-g)) * u).astype(np.float16).astype(np.float64)  # the fp16 intermediate
    y = grouped_matmul(host["moe.down.fp8"][e], host["moe.down.fp8_s"][e], act, fold_scale=False)
    ref = orc.expert_forward(host, e, x, np.float64)
    assert not y[3].any() and not ref[3].any()
    live = [0, 1, 2, 4, 5]
    rel = np.linalg.norm(y[live] - ref[live], axis=1) / np.linalg.norm(ref[live], axis=1)
    assert np.isfinite(rel).all() and rel.max() <= 5e-4, rel
