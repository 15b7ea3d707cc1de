// Attention backward pre-pass: delta[b, h, s] = sum_d O[b, s, h, d] * dO[b, s, h, d] in fp32
// (reference: `flash_bwd_prep`, attention_engine/core/template/tl_template/attn/attn_tl.py:196-223).
// HBM-bound: one warp per row, each lane reads 32-bit pairs so a warp covers 128 B per load.
// Expects AE_DV and AE_BF16.

extern "C" __global__ void __launch_bounds__(256) ae_attn_bwd_prep(const AeAttnBwdPrepArgs args) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int s = blockIdx.x * 8 + warp;
  const int h = blockIdx.y, b = blockIdx.z;
  if (s >= args.Sq) return;
  const u32* o = (const u32*)((const u16*)args.o + (i64)b * args.o_sb + (i64)s * args.o_ss + (i64)h * args.o_sh);
  const u32* d = (const u32*)((const u16*)args.d_o + (i64)b * args.do_sb + (i64)s * args.do_ss + (i64)h * args.do_sh);
  float acc = 0.f;
#pragma unroll
  for (int k = 0; k < AE_DV / 64; ++k) {
    const u32 a = o[k * 32 + lane], c = d[k * 32 + lane];
    acc += unpack_lo<AE_BF16>(a) * unpack_lo<AE_BF16>(c) + unpack_hi<AE_BF16>(a) * unpack_hi<AE_BF16>(c);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) args.delta[((i64)b * args.Hq + h) * args.Sq + s] = acc;
}
