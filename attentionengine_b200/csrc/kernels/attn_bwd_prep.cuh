// Attention backward pre-pass: delta[b, h, s] = sum_d O[b, s, h, d] * dO[b, s, h, d] in fp32
// (reference: `flash_bwd_prep`, attention_engine/core/template/tl_template/attn/attn_tl.py:196-223).
// HBM-bound.  A row is shared by AE_DV / 8 lanes (16 bytes per lane and tensor); rows are taken in (batch, position,
// head) order, the order they lie in memory, four row groups per warp and iteration so that eight 16-byte loads per lane
// are in flight; the CTAs stride over the rows.
// Expects AE_DV (a multiple of 64, at most 256) and AE_BF16.

#define AE_PREP_TPR (AE_DV / 8)         // lanes per row
#define AE_PREP_RPW (32 / AE_PREP_TPR)  // rows per warp and load
#define AE_PREP_UNROLL 4
#if AE_DV != 64 && AE_DV != 128 && AE_DV != 256
#error "value head dim must be 64, 128 or 256"
#endif

extern "C" __global__ void __launch_bounds__(256) ae_attn_bwd_prep(const AeAttnBwdPrepArgs args) {
  const int lane = threadIdx.x & 31;
  const i64 warp0 = ((i64)blockIdx.x * 256 + threadIdx.x) >> 5;
  const i64 n_warps = ((i64)gridDim.x * 256) >> 5;
  const i64 n_rows = (i64)args.B * args.Sq * args.Hq;
  const int sub = lane / AE_PREP_TPR, col = (lane % AE_PREP_TPR) * 8;
  for (i64 base = warp0 * (AE_PREP_RPW * AE_PREP_UNROLL); base < n_rows; base += n_warps * (AE_PREP_RPW * AE_PREP_UNROLL)) {
    uint4 ov[AE_PREP_UNROLL], dv[AE_PREP_UNROLL];
    i64 dst[AE_PREP_UNROLL];
#pragma unroll
    for (int u = 0; u < AE_PREP_UNROLL; ++u) {
      const i64 row = base + u * AE_PREP_RPW + sub;  // (b, s, h) with h fastest
      dst[u] = -1;
      ov[u] = make_uint4(0, 0, 0, 0);
      dv[u] = make_uint4(0, 0, 0, 0);
      if (row < n_rows) {
        const int h = (int)(row % args.Hq);
        const i64 bs = row / args.Hq;
        const int s = (int)(bs % args.Sq), b = (int)(bs / args.Sq);
        ov[u] = *(const uint4*)((const u16*)args.o + (i64)b * args.o_sb + (i64)s * args.o_ss + (i64)h * args.o_sh + col);
        dv[u] = *(const uint4*)((const u16*)args.d_o + (i64)b * args.do_sb + (i64)s * args.do_ss + (i64)h * args.do_sh + col);
        dst[u] = ((i64)b * args.Hq + h) * args.Sq + s;
      }
    }
#pragma unroll
    for (int u = 0; u < AE_PREP_UNROLL; ++u) {
      const u32 a[4] = {ov[u].x, ov[u].y, ov[u].z, ov[u].w}, c[4] = {dv[u].x, dv[u].y, dv[u].z, dv[u].w};
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i)
        acc += unpack_lo<AE_BF16>(a[i]) * unpack_lo<AE_BF16>(c[i]) + unpack_hi<AE_BF16>(a[i]) * unpack_hi<AE_BF16>(c[i]);
#pragma unroll
      for (int off = AE_PREP_TPR / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
      if (dst[u] >= 0 && (lane % AE_PREP_TPR) == 0) args.delta[dst[u]] = acc;
    }
  }
}
