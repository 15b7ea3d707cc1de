// Split-KV merge for the MLA decode (reference: `combine` prim_func, mla_decode_tl.py:181-216; CuTe
// variant cute_template_kvshared/kernels/mla_combine.cu:14-152).  One warp per (batch, head): lane k holds
// the final row scales of split k (n_split <= 32; absent splits hold -inf), the traced
// OnlineFunc.combine runs with its reductions over the split dimension as warp-shuffle reductions and
// leaves each lane with the weight of its split; the lanes then sweep the value dims with 128-bit
// loads, fetching each split's weight by shuffle.
// Expects AE_BF16, AE_NFINAL and ae_combine(const float* fr_of_this_lane) -> weight of this lane's split.

AE_DEVICE float ae_warp_max(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
  return x;
}
AE_DEVICE float ae_warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

//%%AE_COMBINE_FUNCTOR%%

extern "C" __global__ void __launch_bounds__(128) ae_mla_combine(const AeMlaCombineArgs args) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x * 4 + warp;
  const int b = blockIdx.y;
  if (h >= args.H) return;  // warp-uniform
  const int n_split = args.part_off ? args.part_off[b + 1] - args.part_off[b] : args.n_split;
  const i64 slot0 = args.part_off ? (i64)args.part_off[b] : (i64)b * args.n_split;
  if (args.part_off && n_split <= 1) return;  // written directly by the split kernel
  float fr[AE_NFINAL > 0 ? AE_NFINAL : 1];
#pragma unroll
  for (int i = 0; i < AE_NFINAL; ++i)
    fr[i] = lane < n_split ? args.fr_part[i][(slot0 + lane) * args.H + h] : -__int_as_float(0x7f800000);
  float w = ae_combine(fr);
  if (lane >= n_split) w = 0.f;
  u16* orow = (u16*)args.o + ((i64)b * args.H + h) * args.DV;
  // the loop bounds are warp-uniform: every lane takes part in the shuffles, also when DV < 128 leaves it no columns
  for (int base = 0; base < args.DV; base += 128) {
    const int d0 = base + lane * 4;
    const bool active = d0 < args.DV;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < n_split; ++k) {
      const float wk = __shfl_sync(0xffffffffu, w, k);
      if (active) {
        const float4 v = *(const float4*)(args.o_part + ((slot0 + k) * args.H + h) * args.DV + d0);
        acc.x += wk * v.x;
        acc.y += wk * v.y;
        acc.z += wk * v.z;
        acc.w += wk * v.w;
      }
    }
    if (active) {
      uint2 o2;
      o2.x = pack2<AE_BF16>(acc.x, acc.y);
      o2.y = pack2<AE_BF16>(acc.z, acc.w);
      *(uint2*)(orow + d0) = o2;
    }
  }
}
