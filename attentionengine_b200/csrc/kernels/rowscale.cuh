// Row-scale mod of the linear-attention engine and its backward, as two streaming kernels:
//   forward   y[r, :] = x[r, :] * s[r]
//   backward  gx[r, :] = g[r, :] * s[r],   gs[r] = sum_d g[r, d] * x[r, d]
// x, y, g, gx are [n_rows, AE_RS_D] 16-bit, s / gs one value per row (fp32, or the 16-bit type when AE_RS_S16).
// This is the shape of `v_mod = v * dt` of the reference's Mamba2 script (attn_script/mamba2_ngroup1.py:31-33), which
// the reference runs as eager PyTorch statements (core/template/tl_template/linear/linear_tl.py:1136-1144, backward
// :1203-1214); a broadcast multiply and a reduction over 64 contiguous elements are what PyTorch's generic kernels do
// worst (measured 3 to 5 times the time of the bytes moved).
// A row is shared by AE_RS_D / 8 lanes (16 bytes per lane); the loop bounds are warp-uniform so that the shuffles of the
// row reduction are always executed by all 32 lanes.
// Expects AE_BF16, AE_RS_D (64, 128 or 256), AE_RS_S16.
//
// The same file holds the per-head skip connection of the Mamba2 block (o += D_skip[h] * x, the benchmark's config 4;
// the reference's harness passes D=None, benchmark/bench_utils.py:304-308), for rows ordered (batch, head, step):
//   forward   y[r, :] = o[r, :] + x[r, :] * d[head(r)]                      (ae_skip_fwd:  o arrives in `g`)
//   backward  gx[r, :] = g[r, :] * d[head(r)],  gs[r] = sum_d g[r, d] * x[r, d]   (ae_skip_bwd: gs is fp32; the caller
//             sums it over batch and steps to get the gradient of d)
// with head(r) = (r / rows_per_head) % n_heads and d [n_heads] fp32 in `s`.

//
// And the two backward passes of a block that uses both (v' = x * s[row] into the scan, y = o + x * d[head] after it), as
// one pass over x:   gx[r, :] = g2[r, :] * s[r] + g[r, :] * d[head(r)],   gs[r] = sum_d g2 * x,   gs2[r] = sum_d g * x
// with g the gradient of y and g2 the gradient of v' (ae_vskip_bwd): x is read once, and the sum of the two
// contributions to gx needs no pass of its own.

#define AE_RS_TPR (AE_RS_D / 8)        // lanes per row
#define AE_RS_RPW (32 / AE_RS_TPR)     // rows per warp and iteration
#if AE_RS_D != 64 && AE_RS_D != 128 && AE_RS_D != 256
#error "row length must be 64, 128 or 256"
#endif

AE_DEVICE float ae_rs_load_s(const void* s, i64 row) {
#if AE_RS_S16
  return unpack_lo<AE_BF16>((u32)((const u16*)s)[row]);
#else
  return ((const float*)s)[row];
#endif
}

extern "C" __global__ void __launch_bounds__(256) ae_rowscale_fwd(const AeRowScaleArgs a) {
  const int lane = threadIdx.x & 31;
  const i64 warp0 = ((i64)blockIdx.x * 256 + threadIdx.x) >> 5;
  const i64 n_warps = ((i64)gridDim.x * 256) >> 5;
  for (i64 base = warp0 * AE_RS_RPW; base < a.n_rows; base += n_warps * AE_RS_RPW) {
    const i64 row = base + lane / AE_RS_TPR;
    if (row < a.n_rows) {
      const i64 off = row * AE_RS_D + (lane % AE_RS_TPR) * 8;
      const uint4 v = *(const uint4*)((const u16*)a.x + off);
      const float sc = ae_rs_load_s(a.s, row);
      uint4 o;
      o.x = pack2<AE_BF16>(unpack_lo<AE_BF16>(v.x) * sc, unpack_hi<AE_BF16>(v.x) * sc);
      o.y = pack2<AE_BF16>(unpack_lo<AE_BF16>(v.y) * sc, unpack_hi<AE_BF16>(v.y) * sc);
      o.z = pack2<AE_BF16>(unpack_lo<AE_BF16>(v.z) * sc, unpack_hi<AE_BF16>(v.z) * sc);
      o.w = pack2<AE_BF16>(unpack_lo<AE_BF16>(v.w) * sc, unpack_hi<AE_BF16>(v.w) * sc);
      *(uint4*)((u16*)a.y + off) = o;
    }
  }
}

extern "C" __global__ void __launch_bounds__(256) ae_rowscale_bwd(const AeRowScaleArgs a) {
  const int lane = threadIdx.x & 31;
  const i64 warp0 = ((i64)blockIdx.x * 256 + threadIdx.x) >> 5;
  const i64 n_warps = ((i64)gridDim.x * 256) >> 5;
  for (i64 base = warp0 * AE_RS_RPW; base < a.n_rows; base += n_warps * AE_RS_RPW) {
    const i64 row = base + lane / AE_RS_TPR;
    const bool valid = row < a.n_rows;
    float dot = 0.f;
    if (valid) {
      const i64 off = row * AE_RS_D + (lane % AE_RS_TPR) * 8;
      const uint4 g = *(const uint4*)((const u16*)a.g + off);
      const uint4 x = *(const uint4*)((const u16*)a.x + off);
      const float sc = ae_rs_load_s(a.s, row);
      const u32 gw[4] = {g.x, g.y, g.z, g.w}, xw[4] = {x.x, x.y, x.z, x.w};
      u32 ow[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float g0 = unpack_lo<AE_BF16>(gw[i]), g1 = unpack_hi<AE_BF16>(gw[i]);
        dot = fmaf(g0, unpack_lo<AE_BF16>(xw[i]), dot);
        dot = fmaf(g1, unpack_hi<AE_BF16>(xw[i]), dot);
        ow[i] = pack2<AE_BF16>(g0 * sc, g1 * sc);
      }
      *(uint4*)((u16*)a.gx + off) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
#pragma unroll
    for (int o = AE_RS_TPR / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    if (valid && (lane % AE_RS_TPR) == 0) {
#if AE_RS_S16
      ((u16*)a.gs)[row] = (u16)(pack2<AE_BF16>(dot, 0.f) & 0xffffu);
#else
      ((float*)a.gs)[row] = dot;
#endif
    }
  }
}

AE_DEVICE float ae_rs_head_scale(const AeRowScaleArgs& a, i64 row) {
  return ((const float*)a.s)[(row / a.rows_per_head) % a.n_heads];
}

extern "C" __global__ void __launch_bounds__(256) ae_skip_fwd(const AeRowScaleArgs a) {
  const int lane = threadIdx.x & 31;
  const i64 warp0 = ((i64)blockIdx.x * 256 + threadIdx.x) >> 5;
  const i64 n_warps = ((i64)gridDim.x * 256) >> 5;
  for (i64 base = warp0 * AE_RS_RPW; base < a.n_rows; base += n_warps * AE_RS_RPW) {
    const i64 row = base + lane / AE_RS_TPR;
    if (row < a.n_rows) {
      const i64 off = row * AE_RS_D + (lane % AE_RS_TPR) * 8;
      const uint4 x = *(const uint4*)((const u16*)a.x + off);
      const uint4 o = *(const uint4*)((const u16*)a.g + off);
      const float sc = ae_rs_head_scale(a, row);
      const u32 xw[4] = {x.x, x.y, x.z, x.w}, ow[4] = {o.x, o.y, o.z, o.w};
      u32 yw[4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        yw[i] = pack2<AE_BF16>(fmaf(unpack_lo<AE_BF16>(xw[i]), sc, unpack_lo<AE_BF16>(ow[i])),
                               fmaf(unpack_hi<AE_BF16>(xw[i]), sc, unpack_hi<AE_BF16>(ow[i])));
      *(uint4*)((u16*)a.y + off) = make_uint4(yw[0], yw[1], yw[2], yw[3]);
    }
  }
}

extern "C" __global__ void __launch_bounds__(256) ae_skip_bwd(const AeRowScaleArgs a) {
  const int lane = threadIdx.x & 31;
  const i64 warp0 = ((i64)blockIdx.x * 256 + threadIdx.x) >> 5;
  const i64 n_warps = ((i64)gridDim.x * 256) >> 5;
  for (i64 base = warp0 * AE_RS_RPW; base < a.n_rows; base += n_warps * AE_RS_RPW) {
    const i64 row = base + lane / AE_RS_TPR;
    const bool valid = row < a.n_rows;
    float dot = 0.f;
    if (valid) {
      const i64 off = row * AE_RS_D + (lane % AE_RS_TPR) * 8;
      const uint4 g = *(const uint4*)((const u16*)a.g + off);
      const uint4 x = *(const uint4*)((const u16*)a.x + off);
      const float sc = ae_rs_head_scale(a, row);
      const u32 gw[4] = {g.x, g.y, g.z, g.w}, xw[4] = {x.x, x.y, x.z, x.w};
      u32 ow[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float g0 = unpack_lo<AE_BF16>(gw[i]), g1 = unpack_hi<AE_BF16>(gw[i]);
        dot = fmaf(g0, unpack_lo<AE_BF16>(xw[i]), dot);
        dot = fmaf(g1, unpack_hi<AE_BF16>(xw[i]), dot);
        ow[i] = pack2<AE_BF16>(g0 * sc, g1 * sc);
      }
      *(uint4*)((u16*)a.gx + off) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
#pragma unroll
    for (int o = AE_RS_TPR / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    if (valid && (lane % AE_RS_TPR) == 0) ((float*)a.gs)[row] = dot;
  }
}

extern "C" __global__ void __launch_bounds__(256) ae_vskip_bwd(const AeRowScaleArgs a) {
  const int lane = threadIdx.x & 31;
  const i64 warp0 = ((i64)blockIdx.x * 256 + threadIdx.x) >> 5;
  const i64 n_warps = ((i64)gridDim.x * 256) >> 5;
  for (i64 base = warp0 * AE_RS_RPW; base < a.n_rows; base += n_warps * AE_RS_RPW) {
    const i64 row = base + lane / AE_RS_TPR;
    const bool valid = row < a.n_rows;
    float dot_v = 0.f, dot_o = 0.f;
    if (valid) {
      const i64 off = row * AE_RS_D + (lane % AE_RS_TPR) * 8;
      const uint4 g = *(const uint4*)((const u16*)a.g + off);
      const uint4 g2 = *(const uint4*)((const u16*)a.g2 + off);
      const uint4 x = *(const uint4*)((const u16*)a.x + off);
      const float sc = ae_rs_load_s(a.s, row);
      const float dh = a.d[(row / a.rows_per_head) % a.n_heads];
      const u32 gw[4] = {g.x, g.y, g.z, g.w}, vw[4] = {g2.x, g2.y, g2.z, g2.w}, xw[4] = {x.x, x.y, x.z, x.w};
      u32 ow[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float g0 = unpack_lo<AE_BF16>(gw[i]), g1 = unpack_hi<AE_BF16>(gw[i]);
        const float v0 = unpack_lo<AE_BF16>(vw[i]), v1 = unpack_hi<AE_BF16>(vw[i]);
        const float x0 = unpack_lo<AE_BF16>(xw[i]), x1 = unpack_hi<AE_BF16>(xw[i]);
        dot_v = fmaf(v0, x0, dot_v);
        dot_v = fmaf(v1, x1, dot_v);
        dot_o = fmaf(g0, x0, dot_o);
        dot_o = fmaf(g1, x1, dot_o);
        ow[i] = pack2<AE_BF16>(fmaf(v0, sc, g0 * dh), fmaf(v1, sc, g1 * dh));
      }
      *(uint4*)((u16*)a.gx + off) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
#pragma unroll
    for (int o = AE_RS_TPR / 2; o > 0; o >>= 1) {
      dot_v += __shfl_xor_sync(0xffffffffu, dot_v, o);
      dot_o += __shfl_xor_sync(0xffffffffu, dot_o, o);
    }
    if (valid && (lane % AE_RS_TPR) == 0) {
#if AE_RS_S16
      ((u16*)a.gs)[row] = (u16)(pack2<AE_BF16>(dot_v, 0.f) & 0xffffu);
#else
      ((float*)a.gs)[row] = dot_v;
#endif
      a.gs2[row] = dot_o;
    }
  }
}

// Sum over the heads of a group: x [n_groups, G, T, AE_RS_D] 16-bit -> y [n_groups, T, AE_RS_D] 16-bit, fp32 accumulation
// (n_rows = n_groups * T output rows, rows_per_head = T, n_heads = G).  The reverse pass of the scan writes dq / dk per
// value head; q and k may have fewer heads (the reference sums the same way, linear_tl.py:1198-1201).
extern "C" __global__ void __launch_bounds__(256) ae_head_sum(const AeRowScaleArgs a) {
  const int lane = threadIdx.x & 31;
  const i64 warp0 = ((i64)blockIdx.x * 256 + threadIdx.x) >> 5;
  const i64 n_warps = ((i64)gridDim.x * 256) >> 5;
  const i64 T = a.rows_per_head;
  const int G = a.n_heads;
  for (i64 base = warp0 * AE_RS_RPW; base < a.n_rows; base += n_warps * AE_RS_RPW) {
    const i64 row = base + lane / AE_RS_TPR;
    if (row < a.n_rows) {
      const i64 grp = row / T, t = row - grp * T;
      const u16* src = (const u16*)a.x + ((grp * G) * T + t) * AE_RS_D + (lane % AE_RS_TPR) * 8;
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
      int g = 0;
      for (; g + 4 <= G; g += 4) {  // four independent 16-byte loads in flight per lane
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = *(const uint4*)(src + (i64)(g + u) * T * AE_RS_D);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const u32 w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            acc[2 * i] += unpack_lo<AE_BF16>(w[i]);
            acc[2 * i + 1] += unpack_hi<AE_BF16>(w[i]);
          }
        }
      }
      for (; g < G; ++g) {
        const uint4 v = *(const uint4*)(src + (i64)g * T * AE_RS_D);
        const u32 w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          acc[2 * i] += unpack_lo<AE_BF16>(w[i]);
          acc[2 * i + 1] += unpack_hi<AE_BF16>(w[i]);
        }
      }
      uint4 o;
      o.x = pack2<AE_BF16>(acc[0], acc[1]);
      o.y = pack2<AE_BF16>(acc[2], acc[3]);
      o.z = pack2<AE_BF16>(acc[4], acc[5]);
      o.w = pack2<AE_BF16>(acc[6], acc[7]);
      *(uint4*)((u16*)a.y + row * AE_RS_D + (lane % AE_RS_TPR) * 8) = o;
    }
  }
}
