// hy_attn.cuh — tensor-core attention of the layered hybrid decoders (bf16 build): causal softmax attention with a sink
// whose values are its keys, over the paged key cache, for prompt portions and decoded tokens alike.
//
// Work unit = (entry, key head, tile of 64 query rows, key split).  The rows of a tile are (token, query head of the
// group) pairs, token-major, so the R = heads / kv_heads query heads that share a key head also share every key tile that
// is loaded.  A unit walks its key range in tiles of 64 keys aligned to absolute positions:
//   S = Q K^T      mma.sync m16n8k16 bf16, fp32 accumulators; the score is scaled by scale * temperature(position) in fp32
//   online softmax in fp32 (running maximum and sum per row)
//   O += P K       the weights stay 32-bit in effect: P is split into a bf16 head and a bf16 remainder, two products
// and leaves unnormalised partial results (m, l, O) per (row, split).  The combine kernel merges the splits of a row with
// the sink (a logit with no key and no value: it only enters the maximum and the denominator), applies the output gate
// and the mixer's scale and writes the operand of the output projection.
#pragma once
#include "hy_kernels.cuh"
#include "jf_ptx.cuh"

namespace hy {

struct AttnUnit { int entry, kv_head, row0, split; };   // row0: first row of the tile inside the entry (rows = tokens x R)

template <int DIM>
__global__ void __launch_bounds__(128) attn_mma_kernel(Batch b, const AttnUnit* __restrict__ units, const bf16* __restrict__ q,
                                                       int ldq, const bf16* __restrict__ cache, int H, int G, float scale,
                                                       float qt_coef, int qt_every, int split_keys, int n_splits, int vdim,
                                                       float* __restrict__ part_o, float* __restrict__ part_ml) {
  constexpr int LD = DIM + 8;                           // padded row (elements): ldmatrix rows fall into distinct banks
  __shared__ __align__(16) bf16 qs[64 * LD];
  __shared__ __align__(16) bf16 ks[64 * LD];
  const AttnUnit u = units[blockIdx.x];
  const int R = H / G;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int start = b.ent_start[u.entry], cnt = b.ent_start[u.entry + 1] - start, pos0 = b.ent_pos0[u.entry];
  const int rows_total = cnt * R;
  const int* pg = b.pages + (size_t)u.entry * b.max_pages;
  // ---- the query tile: row r -> token start + (row0 + r) / R, head kv_head * R + (row0 + r) % R ------------------------
  for (int i = tid; i < 64 * (DIM / 8); i += 128) {
    const int r = i / (DIM / 8), c = i % (DIM / 8);
    const int row = u.row0 + r;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < rows_total)
      v = *reinterpret_cast<const uint4*>(q + (size_t)(start + row / R) * ldq + (u.kv_head * R + row % R) * DIM + c * 8);
    *reinterpret_cast<uint4*>(&qs[r * LD + c * 8]) = v;
  }
  __syncthreads();
  uint32_t qa[DIM / 16][4];
  {
    const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
    for (int kk = 0; kk < DIM / 16; ++kk)
      jf::ldmatrix_x4(jf::smem_u32(&qs[r * LD + kk * 16 + (lane >> 4) * 8]), qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3]);
  }
  // this thread's two rows
  const int r_lo = u.row0 + warp * 16 + (lane >> 2), r_hi = r_lo + 8;
  const bool v_lo = r_lo < rows_total, v_hi = r_hi < rows_total;
  const int p_lo = v_lo ? pos0 + r_lo / R : -1, p_hi = v_hi ? pos0 + r_hi / R : -1;
  const float f_lo = scale * (1.0f + qt_coef * logf(floorf((float)(p_lo + 1) / (float)qt_every) + 1.0f));
  const float f_hi = scale * (1.0f + qt_coef * logf(floorf((float)(p_hi + 1) / (float)qt_every) + 1.0f));
  const bool warp_live = (u.row0 + warp * 16) < rows_total;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.0f, l_hi = 0.0f;
  float o[DIM / 8][4];
#pragma unroll
  for (int i = 0; i < DIM / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
  // key range of this unit: its split, cut at the last position any row of the tile may see
  const int last_row = min(u.row0 + 63, rows_total - 1);
  const int key_end = min((u.split + 1) * split_keys, pos0 + last_row / R + 1);
  for (int j0 = u.split * split_keys; j0 < key_end; j0 += 64) {
    __syncthreads();                                     // the previous tile has been read
    for (int i = tid; i < 64 * (DIM / 8); i += 128) {
      const int r = i / (DIM / 8), c = i % (DIM / 8);
      const int j = j0 + r;
      const bool ok = j < key_end;
      const int jj = ok ? j : j0;
      const bf16* src = cache + (((size_t)pg[jj / b.page_size] * G + u.kv_head) * b.page_size + jj % b.page_size) * DIM + c * 8;
      jf::cp_async_16(&ks[r * LD + c * 8], src, ok ? 16u : 0u);
    }
    jf::cp_async_commit();
    jf::cp_async_wait_all();
    __syncthreads();
    if (!warp_live) continue;
    // ---- scores: 16 rows x 64 keys per warp -------------------------------------------------------------------------
    float s[8][4];
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) { s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.0f; }
#pragma unroll
    for (int kk = 0; kk < DIM / 16; ++kk) {
#pragma unroll
      for (int np = 0; np < 4; ++np) {                   // two key blocks of 8 per ldmatrix
        uint32_t b0, b1, b2, b3;
        const int key = np * 16 + (lane & 7) + (lane >> 4) * 8;
        jf::ldmatrix_x4(jf::smem_u32(&ks[key * LD + kk * 16 + ((lane >> 3) & 1) * 8]), b0, b1, b2, b3);
        jf::mma_bf16_16816(s[np * 2], qa[kk], b0, b1);
        jf::mma_bf16_16816(s[np * 2 + 1], qa[kk], b2, b3);
      }
    }
    // ---- mask, scale, running maximum -----------------------------------------------------------------------------------
    float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int j = j0 + nb * 8 + (lane & 3) * 2 + c;
        s[nb][c] = (j <= p_lo && j < key_end) ? s[nb][c] * f_lo : -INFINITY;
        s[nb][2 + c] = (j <= p_hi && j < key_end) ? s[nb][2 + c] * f_hi : -INFINITY;
        mx_lo = fmaxf(mx_lo, s[nb][c]);
        mx_hi = fmaxf(mx_hi, s[nb][2 + c]);
      }
    }
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
    const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
    const float ref_lo = mn_lo == -INFINITY ? 0.0f : mn_lo, ref_hi = mn_hi == -INFINITY ? 0.0f : mn_hi;
    const float c_lo = expf(m_lo - ref_lo), c_hi = expf(m_hi - ref_hi);      // m = -inf: exp(-inf) = 0
    m_lo = mn_lo; m_hi = mn_hi;
    float sum_lo = 0.0f, sum_hi = 0.0f;
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        s[nb][c] = expf(s[nb][c] - ref_lo);
        s[nb][2 + c] = expf(s[nb][2 + c] - ref_hi);
        sum_lo += s[nb][c];
        sum_hi += s[nb][2 + c];
      }
    }
    sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 1);
    sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 2);
    sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 1);
    sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 2);
    l_lo = l_lo * c_lo + sum_lo;
    l_hi = l_hi * c_hi + sum_hi;
#pragma unroll
    for (int i = 0; i < DIM / 8; ++i) { o[i][0] *= c_lo; o[i][1] *= c_lo; o[i][2] *= c_hi; o[i][3] *= c_hi; }
    // ---- O += P K: P as a bf16 head plus a bf16 remainder ----------------------------------------------------------------
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {                     // 16 keys per step
      uint32_t ph[4], pl[4];
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const float* sv = s[kk * 2 + half];
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
          const float x0 = sv[rr * 2], x1 = sv[rr * 2 + 1];
          const float h0 = jf::bf16_round(x0), h1 = jf::bf16_round(x1);
          ph[half * 2 + rr] = jf::pack_bf16x2(h0, h1);
          pl[half * 2 + rr] = jf::pack_bf16x2(x0 - h0, x1 - h1);
        }
      }
#pragma unroll
      for (int np = 0; np < DIM / 16; ++np) {            // two dim blocks of 8 per ldmatrix; values: the first vdim dims
        if (np * 16 >= vdim) continue;
        uint32_t b0, b1, b2, b3;
        const int key = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        jf::ldmatrix_x4_trans(jf::smem_u32(&ks[key * LD + np * 16 + (lane >> 4) * 8]), b0, b1, b2, b3);
        jf::mma_bf16_16816(o[np * 2], ph, b0, b1);
        jf::mma_bf16_16816(o[np * 2], pl, b0, b1);
        jf::mma_bf16_16816(o[np * 2 + 1], ph, b2, b3);
        jf::mma_bf16_16816(o[np * 2 + 1], pl, b2, b3);
      }
    }
  }
  // ---- partial results ---------------------------------------------------------------------------------------------------------
  if (!warp_live) return;
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    const int row = hh ? r_hi : r_lo;
    if (row >= rows_total) continue;
    const int t = start + row / R, h = u.kv_head * R + row % R;
    const size_t slot = ((size_t)t * H + h) * n_splits + u.split;
    float* po = part_o + slot * DIM;
#pragma unroll
    for (int i = 0; i < DIM / 8; ++i)
      *reinterpret_cast<float2*>(po + i * 8 + (lane & 3) * 2) = make_float2(o[i][hh * 2], o[i][hh * 2 + 1]);
    if ((lane & 3) == 0) {
      part_ml[slot * 2] = hh ? m_hi : m_lo;
      part_ml[slot * 2 + 1] = hh ? l_hi : l_lo;
    }
  }
}


// ---- the same attention for wide cache rows (one key head, rows of up to 640 elements, values = the first vdim <= 512) ------
// Serves attention over a shared latent at the sizes real models use (rank 512 + 64 rotated): a (token, head) row keeps
// vdim output values, too many for the 16 rows x all values per warp of the kernel above.  Eight warps share a tile of
// 64 rows x 64 keys in two phases:
//   scores   warp w: rows 16 (w % 4) .., keys 32 (w / 4) ..; Q and K fragments both come from shared memory
//   softmax  row maxima and sums meet in shared memory (two warps share a row); the weights go to shared memory as a bf16
//            head and a bf16 remainder
//   values   warp w: ALL 64 rows x value dimensions [w NT 8, (w + 1) NT 8): O += P K[:, those dimensions]
// Rows of the tile beyond the entry's rows cost nothing in the value phase (decode steps fill a fraction of a tile).
// Unnormalised partial results (m, l, O) per (row, split) as above; part_o rows are pstride wide.
template <int NT>
__global__ void __launch_bounds__(256, 1) attn_wide_kernel(Batch b, const AttnUnit* __restrict__ units, const bf16* __restrict__ q,
                                                           int ldq, const bf16* __restrict__ cache, int H, int dk, int vdim,
                                                           float scale, int split_keys, int n_splits, int pstride,
                                                           float* __restrict__ part_o, float* __restrict__ part_ml) {
  extern __shared__ __align__(16) unsigned char hy_smem[];
  const int dkp = (dk + 15) & ~15, LD = dkp + 8;          // padded row (elements): ldmatrix rows fall into distinct banks
  constexpr int LDP = 64 + 8;
  bf16* qs = reinterpret_cast<bf16*>(hy_smem);            // [64][LD]
  bf16* ks = qs + 64 * LD;                                // [64][LD]
  bf16* ph = ks + 64 * LD;                                // [64][LDP] weights, bf16 head
  bf16* pl = ph + 64 * LDP;                               // [64][LDP] weights, bf16 remainder
  float* pmax = reinterpret_cast<float*>(pl + 64 * LDP);  // [2][64]
  float* psum = pmax + 128;                               // [2][64]
  float* m_run = psum + 128;                              // [64]
  float* l_run = m_run + 64;                              // [64]
  float* corr = l_run + 64;                               // [64]
  const AttnUnit u = units[blockIdx.x];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int start = b.ent_start[u.entry], cnt = b.ent_start[u.entry + 1] - start, pos0 = b.ent_pos0[u.entry];
  const int rows_total = cnt * H;
  const int rows_here = min(64, rows_total - u.row0);
  const int live_mt = (rows_here + 15) >> 4;
  const int* pg = b.pages + (size_t)u.entry * b.max_pages;
  const int chunks = dk / 8;                              // 16-byte pieces of a row (dk is a multiple of 8)
  for (int i = tid; i < 64 * (LD / 8); i += 256) {        // zero both tiles once: padding columns stay zero
    const int r = i / (LD / 8), c = i % (LD / 8);
    *reinterpret_cast<uint4*>(&qs[r * LD + c * 8]) = make_uint4(0, 0, 0, 0);
    *reinterpret_cast<uint4*>(&ks[r * LD + c * 8]) = make_uint4(0, 0, 0, 0);
  }
  if (tid < 64) { m_run[tid] = -INFINITY; l_run[tid] = 0.0f; }
  __syncthreads();
  for (int i = tid; i < 64 * chunks; i += 256) {
    const int r = i / chunks, c = i % chunks;
    const int row = u.row0 + r;
    if (row < rows_total)
      *reinterpret_cast<uint4*>(&qs[r * LD + c * 8]) =
          *reinterpret_cast<const uint4*>(q + (size_t)(start + row / H) * ldq + (row % H) * dk + c * 8);
  }
  // scores: this thread's two rows and its warp's 32 keys
  const int sm_t = warp & 3, sk0 = (warp >> 2) * 32;
  const int r_lo = sm_t * 16 + (lane >> 2), r_hi = r_lo + 8;
  const bool v_lo = u.row0 + r_lo < rows_total, v_hi = u.row0 + r_hi < rows_total;
  const int p_lo = v_lo ? pos0 + (u.row0 + r_lo) / H : -1, p_hi = v_hi ? pos0 + (u.row0 + r_hi) / H : -1;
  const bool s_live = sm_t < live_mt;
  float o[4][NT][4];
#pragma unroll
  for (int mt = 0; mt < 4; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) { o[mt][nt][0] = o[mt][nt][1] = o[mt][nt][2] = o[mt][nt][3] = 0.0f; }
  const int last_row = min(u.row0 + 63, rows_total - 1);
  const int key_end = min((u.split + 1) * split_keys, pos0 + last_row / H + 1);
  const int d0 = warp * NT * 8;                           // this warp's value dimensions
  for (int j0 = u.split * split_keys; j0 < key_end; j0 += 64) {
    __syncthreads();                                      // the previous tile (keys and weights) has been read
    for (int i = tid; i < 64 * chunks; i += 256) {
      const int r = i / chunks, c = i % chunks;
      const int j = j0 + r;
      const bool ok = j < key_end;
      const int jj = ok ? j : j0;
      const bf16* src = cache + ((size_t)pg[jj / b.page_size] * b.page_size + jj % b.page_size) * dk + c * 8;
      jf::cp_async_16(&ks[r * LD + c * 8], src, ok ? 16u : 0u);
    }
    jf::cp_async_commit();
    jf::cp_async_wait_all();
    __syncthreads();
    // ---- scores ------------------------------------------------------------------------------------------------------------
    float s[4][4];
#pragma unroll
    for (int nb = 0; nb < 4; ++nb) { s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.0f; }
    if (s_live) {
      const int qr = sm_t * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
      for (int kk = 0; kk < dkp / 16; ++kk) {
        uint32_t qa[4];
        jf::ldmatrix_x4(jf::smem_u32(&qs[qr * LD + kk * 16 + (lane >> 4) * 8]), qa[0], qa[1], qa[2], qa[3]);
#pragma unroll
        for (int np = 0; np < 2; ++np) {
          uint32_t b0, b1, b2, b3;
          const int key = sk0 + np * 16 + (lane & 7) + (lane >> 4) * 8;
          jf::ldmatrix_x4(jf::smem_u32(&ks[key * LD + kk * 16 + ((lane >> 3) & 1) * 8]), b0, b1, b2, b3);
          jf::mma_bf16_16816(s[np * 2], qa, b0, b1);
          jf::mma_bf16_16816(s[np * 2 + 1], qa, b2, b3);
        }
      }
    }
    float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
    for (int nb = 0; nb < 4; ++nb) {
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int j = j0 + sk0 + nb * 8 + (lane & 3) * 2 + c;
        s[nb][c] = (j <= p_lo && j < key_end) ? s[nb][c] * scale : -INFINITY;
        s[nb][2 + c] = (j <= p_hi && j < key_end) ? s[nb][2 + c] * scale : -INFINITY;
        mx_lo = fmaxf(mx_lo, s[nb][c]);
        mx_hi = fmaxf(mx_hi, s[nb][2 + c]);
      }
    }
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
    if ((lane & 3) == 0) { pmax[(warp >> 2) * 64 + r_lo] = mx_lo; pmax[(warp >> 2) * 64 + r_hi] = mx_hi; }
    __syncthreads();
    {
      const float mn_lo = fmaxf(m_run[r_lo], fmaxf(pmax[r_lo], pmax[64 + r_lo]));
      const float mn_hi = fmaxf(m_run[r_hi], fmaxf(pmax[r_hi], pmax[64 + r_hi]));
      const float ref_lo = mn_lo == -INFINITY ? 0.0f : mn_lo, ref_hi = mn_hi == -INFINITY ? 0.0f : mn_hi;
      float sum_lo = 0.0f, sum_hi = 0.0f;
#pragma unroll
      for (int nb = 0; nb < 4; ++nb) {
        const float a0 = expf(s[nb][0] - ref_lo), a1 = expf(s[nb][1] - ref_lo);
        const float c0 = expf(s[nb][2] - ref_hi), c1 = expf(s[nb][3] - ref_hi);
        sum_lo += a0 + a1;
        sum_hi += c0 + c1;
        const float ah0 = jf::bf16_round(a0), ah1 = jf::bf16_round(a1), ch0 = jf::bf16_round(c0), ch1 = jf::bf16_round(c1);
        const int col = sk0 + nb * 8 + (lane & 3) * 2;
        *reinterpret_cast<uint32_t*>(&ph[r_lo * LDP + col]) = jf::pack_bf16x2(ah0, ah1);
        *reinterpret_cast<uint32_t*>(&pl[r_lo * LDP + col]) = jf::pack_bf16x2(a0 - ah0, a1 - ah1);
        *reinterpret_cast<uint32_t*>(&ph[r_hi * LDP + col]) = jf::pack_bf16x2(ch0, ch1);
        *reinterpret_cast<uint32_t*>(&pl[r_hi * LDP + col]) = jf::pack_bf16x2(c0 - ch0, c1 - ch1);
      }
      sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 1);
      sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 2);
      sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 1);
      sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 2);
      if ((lane & 3) == 0) { psum[(warp >> 2) * 64 + r_lo] = sum_lo; psum[(warp >> 2) * 64 + r_hi] = sum_hi; }
    }
    __syncthreads();
    if (tid < 64) {                                       // running maximum, sum and this tile's correction per row
      const float mo = m_run[tid];
      const float mn = fmaxf(mo, fmaxf(pmax[tid], pmax[64 + tid]));
      const float ref = mn == -INFINITY ? 0.0f : mn;
      const float cf = expf(mo - ref);                    // mo = -inf: 0
      corr[tid] = cf;
      l_run[tid] = l_run[tid] * cf + psum[tid] + psum[64 + tid];
      m_run[tid] = mn;
    }
    __syncthreads();
    // ---- values: O <- corr O + P K[:, d0 ..] ---------------------------------------------------------------------------------
    if (d0 < vdim) {
#pragma unroll
      for (int mt = 0; mt < 4; ++mt) {
        if (mt >= live_mt) continue;
        const float c_lo = corr[mt * 16 + (lane >> 2)], c_hi = corr[mt * 16 + (lane >> 2) + 8];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) { o[mt][nt][0] *= c_lo; o[mt][nt][1] *= c_lo; o[mt][nt][2] *= c_hi; o[mt][nt][3] *= c_hi; }
      }
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {                    // 16 keys per step
        uint32_t vb[NT][2];
#pragma unroll
        for (int np = 0; np < NT / 2; ++np) {
          const int key = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
          jf::ldmatrix_x4_trans(jf::smem_u32(&ks[key * LD + d0 + np * 16 + (lane >> 4) * 8]), vb[np * 2][0], vb[np * 2][1],
                                vb[np * 2 + 1][0], vb[np * 2 + 1][1]);
        }
#pragma unroll
        for (int mt = 0; mt < 4; ++mt) {
          if (mt >= live_mt) continue;
          uint32_t ah[4], al[4];
          const int pr = mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
          jf::ldmatrix_x4(jf::smem_u32(&ph[pr * LDP + kk * 16 + (lane >> 4) * 8]), ah[0], ah[1], ah[2], ah[3]);
          jf::ldmatrix_x4(jf::smem_u32(&pl[pr * LDP + kk * 16 + (lane >> 4) * 8]), al[0], al[1], al[2], al[3]);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            jf::mma_bf16_16816(o[mt][nt], ah, vb[nt][0], vb[nt][1]);
            jf::mma_bf16_16816(o[mt][nt], al, vb[nt][0], vb[nt][1]);
          }
        }
      }
    }
  }
  __syncthreads();
  // ---- partial results ---------------------------------------------------------------------------------------------------------
  if (tid < rows_here) {
    const int row = u.row0 + tid;
    const size_t slot = ((size_t)(start + row / H) * H + row % H) * n_splits + u.split;
    part_ml[slot * 2] = m_run[tid];
    part_ml[slot * 2 + 1] = l_run[tid];
  }
  if (d0 >= vdim) return;
#pragma unroll
  for (int mt = 0; mt < 4; ++mt) {
    if (mt >= live_mt) continue;
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const int r = mt * 16 + (lane >> 2) + hh * 8;
      if (r >= rows_here) continue;
      const int row = u.row0 + r;
      const size_t slot = ((size_t)(start + row / H) * H + row % H) * n_splits + u.split;
      float* po = part_o + slot * pstride + d0;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
        *reinterpret_cast<float2*>(po + nt * 8 + (lane & 3) * 2) = make_float2(o[mt][nt][hh * 2], o[mt][nt][hh * 2 + 1]);
    }
  }
}

constexpr size_t attn_wide_smem(int dk) {
  return (size_t)2 * 64 * (((dk + 15) & ~15) + 8) * 2 + (size_t)2 * 64 * 72 * 2 + (256 + 192) * 4;
}

// Merge the key splits of one (token, head) with the sink, gate the result, scale it, write the projection's operand.
// part_o rows are dim wide; the first vdim of them are values.
template <typename WT, typename OT>
__global__ void attn_combine_kernel(Batch b, const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    const WT* __restrict__ sink, const bf16* __restrict__ gate, int ldg, int H, int dim,
                                    int vdim, int split_keys, int n_splits, float out_scale, OT* __restrict__ out, int ldo) {
  const int t = blockIdx.x / H, h = blockIdx.x % H;
  const int live = b.tok_pos[t] / split_keys + 1;          // splits that hold a key this row may see
  const float sk = to_f(sink[h]);
  const size_t slot0 = ((size_t)t * H + h) * n_splits;
  float M = sk;
  for (int s = 0; s < live; ++s) M = fmaxf(M, part_ml[(slot0 + s) * 2]);
  float L = expf(sk - M);
  for (int s = 0; s < live; ++s) L += part_ml[(slot0 + s) * 2 + 1] * expf(part_ml[(slot0 + s) * 2] - M);
  const float inv = 1.0f / L;
  for (int d = threadIdx.x; d < vdim; d += blockDim.x) {
    float acc = 0.0f;
    for (int s = 0; s < live; ++s) acc += part_o[(slot0 + s) * dim + d] * expf(part_ml[(slot0 + s) * 2] - M);
    const float gt = gate ? sigmoid_f(to_f(gate[(size_t)t * ldg + h * vdim + d])) : 1.0f;
    out[(size_t)t * ldo + h * vdim + d] = from_f<OT>(acc * inv * gt * out_scale);
  }
}

}  // namespace hy
