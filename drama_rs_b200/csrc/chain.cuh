// Workspace of the chained decode sequence (drb_moe_decode_chained), shared by its kernels in moe_decode.cuh.
// Offsets in floats from the workspace base; the caller zeroes the workspace once before the first call.
//
//   acc      [ACC_REPS][ACC_COLS] u64  fixed-point accumulators (block b adds to copy b % ACC_REPS, which spreads the
//                            atomics over more cache lines; the last block sums the copies) of the next layer's router: column c <= e_next collects
//                            sum_n router[c][n] * y[n] * nw[n] (scale 2^24), column e_next + 1 collects sum_n y[n]^2
//                            (scale 2^16). The down blocks add their shares with integer atomics, so the totals do
//                            not depend on the order of arrival; the last block reads them and leaves them zero.
//   counter  u32             arrivals of the down blocks; left zero.
//   route    [ROUTE_REPS][32] idx[8] (int bits), wts[8], sgate, padding: the routing, replicated so that the blocks
//                            of the next kernels do not all read the same cache line at once
//   yrep     [VEC_REPS][2048] the new hidden state, replicated for the same reason
#pragma once

namespace chainws {

constexpr int ACC_COLS = 272;  // >= 256 + 2; 2 * ACC_COLS floats are a multiple of 32
constexpr int ACC_REPS = 8;
constexpr double FX_LOGIT = 16777216.0, FX_SSQ = 65536.0;
constexpr int ROUTE_REPS = 16, ROUTE_STRIDE = 32;
constexpr int VEC_REPS = 4;
constexpr int HID = 2048;
constexpr int OFF_ACC = 0;
constexpr int OFF_COUNTER = OFF_ACC + 2 * ACC_COLS * ACC_REPS;
constexpr int OFF_ROUTE = OFF_COUNTER + 32;
constexpr int OFF_YREP = OFF_ROUTE + ROUTE_REPS * ROUTE_STRIDE;
constexpr int TOTAL_FLOATS = OFF_YREP + VEC_REPS * HID;
static_assert(OFF_ROUTE % 32 == 0 && OFF_YREP % 32 == 0, "128-byte aligned sections");

}  // namespace chainws
