// bk_gemv_dp4a.cuh -- the integer-dot arithmetic of the batch-1 Q4_K x Q8_1 GEMV, shared by the per-op kernel
// (bk_gemv.cu) and the persistent decode-step kernel (bk_persist.cu): unit decode, 16 dp4a per 64 weights, the fixed
// f32 form per unit, the transposed 8-row warp reduction and the bulk-copy request of a row group.
#pragma once
#include "bk_gemv_shared.cuh"

namespace {

struct RowRegs {
  uint4 hdr, qa, qb;
};

__device__ __forceinline__ RowRegs load_unit(const uint8_t* row, int u) {
  const uint8_t* sb = row + (size_t)(u >> 2) * 144;
  RowRegs r;
  r.hdr = __ldg(reinterpret_cast<const uint4*>(sb));
  const uint4* q = reinterpret_cast<const uint4*>(sb + 16 + (u & 3) * 32);
  r.qa = __ldg(q);
  r.qb = __ldg(q + 1);
  return r;
}

// activation of one unit (two Q8_1 blocks) for one batch column
struct XRegs {
  uint4 x0, x1, x2, x3;
  float2 d8, s8;
};

__device__ __forceinline__ XRegs load_x(const uint32_t* xs, const float* d8s, const float* s8s, int b, int u, int nunits,
                                        int nblk) {
  XRegs r;
  const uint4* xv = reinterpret_cast<const uint4*>(xs + (b * nunits + u) * kUnitWords);
  r.x0 = xv[0];
  r.x1 = xv[1];
  r.x2 = xv[2];
  r.x3 = xv[3];
  r.d8 = *reinterpret_cast<const float2*>(d8s + b * nblk + 2 * u);
  r.s8 = *reinterpret_cast<const float2*>(s8s + b * nblk + 2 * u);
  return r;
}

// weights of one unit, decoded once and shared by all batch columns
struct WRegs {
  uint32_t lo[8], hi[8];
  float d, dmin, fm0, fm1;
  int sc0, sc1;
};

__device__ __forceinline__ WRegs decode_unit(const RowRegs& r, int p) {
  WRegs w;
  w.d = bk_f16_to_f32((uint16_t)(r.hdr.x & 0xffffu));
  w.dmin = bk_f16_to_f32((uint16_t)(r.hdr.x >> 16));
  uint32_t sc2, mn2;
  bk_q4k_scale_min_pair(r.hdr.y, r.hdr.z, r.hdr.w, p, sc2, mn2);
  w.sc0 = (int)(sc2 & 0xffu);
  w.sc1 = (int)(sc2 >> 8);
  w.fm0 = (float)(int)(mn2 & 0xffu);
  w.fm1 = (float)(int)(mn2 >> 8);
  const uint32_t qw[8] = {r.qa.x, r.qa.y, r.qa.z, r.qa.w, r.qb.x, r.qb.y, r.qb.z, r.qb.w};
#pragma unroll
  for (int k = 0; k < 8; k++) {
    w.lo[k] = qw[k] & 0x0f0f0f0fu;
    w.hi[k] = qw[k] & 0xf0f0f0f0u;   // high nibbles stay in place: unsigned bytes 16*q, the staged d8 of odd blocks carries 1/16
  }
  return w;
}

__device__ __forceinline__ float unit_val(const WRegs& w, const XRegs& x) {
  int i0 = 0, i1 = 0;
  i0 = bk_dp4a(w.lo[0], x.x0.x, i0);
  i0 = bk_dp4a(w.lo[1], x.x0.y, i0);
  i0 = bk_dp4a(w.lo[2], x.x0.z, i0);
  i0 = bk_dp4a(w.lo[3], x.x0.w, i0);
  i0 = bk_dp4a(w.lo[4], x.x1.x, i0);
  i0 = bk_dp4a(w.lo[5], x.x1.y, i0);
  i0 = bk_dp4a(w.lo[6], x.x1.z, i0);
  i0 = bk_dp4a(w.lo[7], x.x1.w, i0);
  i1 = bk_dp4a(w.hi[0], x.x2.x, i1);
  i1 = bk_dp4a(w.hi[1], x.x2.y, i1);
  i1 = bk_dp4a(w.hi[2], x.x2.z, i1);
  i1 = bk_dp4a(w.hi[3], x.x2.w, i1);
  i1 = bk_dp4a(w.hi[4], x.x3.x, i1);
  i1 = bk_dp4a(w.hi[5], x.x3.y, i1);
  i1 = bk_dp4a(w.hi[6], x.x3.z, i1);
  i1 = bk_dp4a(w.hi[7], x.x3.w, i1);
  // i1 = 16 * (sub-block sum): sc1*i1 < 2^26 is a multiple of 16, exact in f32, and x.d8.y = d8/16 (exact), so the
  // fma rounds the same real number as fma(d8, f32(sc1*sum), accd)
  float accd = __fmul_rn(x.d8.x, (float)(w.sc0 * i0));
  accd = fmaf(x.d8.y, (float)(w.sc1 * i1), accd);
  float accm = __fmul_rn(x.s8.x, w.fm0);
  accm = fmaf(x.s8.y, w.fm1, accm);
  const float t = __fmul_rn(w.dmin, accm);
  return fmaf(w.d, accd, -t);
}

__device__ __forceinline__ RowRegs load_unit_smem(const uint8_t* row, int u) {
  const uint8_t* sb = row + (size_t)(u >> 2) * 144;
  RowRegs r;
  r.hdr = *reinterpret_cast<const uint4*>(sb);
  const uint4* q = reinterpret_cast<const uint4*>(sb + 16 + (u & 3) * 32);
  r.qa = q[0];
  r.qb = q[1];
  return r;
}

// Sum 8 per-lane values over the warp with 9 shuffles instead of 40: at each of the first three
// levels a lane keeps half of its values and trades the other half with its xor partner.  Every
// addition is one the 16,8,4,2,1 butterfly would make, so the bits are the butterfly's.
// On return lane l holds the total of value index 4*bit4(l) + 2*bit3(l) + bit2(l).
__device__ __forceinline__ float warp_sum8(const float (&v)[8]) {
  const int lane = threadIdx.x & 31;
  const bool b4 = lane & 16, b3 = lane & 8, b2 = lane & 4;
  float w[4], x[2];
#pragma unroll
  for (int i = 0; i < 4; i++) {
    float send = b4 ? v[i] : v[i + 4];
    float keep = b4 ? v[i + 4] : v[i];
    w[i] = __fadd_rn(keep, __shfl_xor_sync(0xffffffffu, send, 16));
  }
#pragma unroll
  for (int i = 0; i < 2; i++) {
    float send = b3 ? w[i] : w[i + 2];
    float keep = b3 ? w[i + 2] : w[i];
    x[i] = __fadd_rn(keep, __shfl_xor_sync(0xffffffffu, send, 8));
  }
  float send = b2 ? x[0] : x[1];
  float keep = b2 ? x[1] : x[0];
  float y = __fadd_rn(keep, __shfl_xor_sync(0xffffffffu, send, 4));
  y = __fadd_rn(y, __shfl_xor_sync(0xffffffffu, y, 2));
  y = __fadd_rn(y, __shfl_xor_sync(0xffffffffu, y, 1));
  return y;
}

// Request the nr rows of a group (first virtual row v0) into its slot.  Rows that follow each other inside one
// matrix are contiguous in memory, so a run of them is ONE bulk copy; a SwiGLU group is two runs (its gate rows,
// then its up rows), which is why its rows sit in the slot as [gate rows | up rows] (see slot_row()).
__device__ __forceinline__ void request_group(const GemvParams& p, int v0, int nr, uint32_t rowb, uint32_t dst, uint32_t bar) {
  mbar_expect_tx(bar, nr * rowb);
  const VRow first = decode_vrow(p, v0);
  const SegDev& sg = p.segs[first.si];
  if (sg.epi == BK_EPI_SWIGLU) {
    const int half = nr >> 1;
    bulk_g2s(dst, sg.W + (size_t)rowb * first.n, half * rowb, bar);
    bulk_g2s(dst + half * rowb, sg.W2 + (size_t)rowb * first.n, half * rowb, bar);
    return;
  }
  int done = 0;
  while (done < nr) {  // one iteration unless the group straddles a segment boundary
    const VRow vr = decode_vrow(p, v0 + done);
    const SegDev& s2 = p.segs[vr.si];
    int run = s2.n_rows - vr.n;
    if (run > nr - done) run = nr - done;
    bulk_g2s(dst + done * rowb, vr.row, run * rowb, bar);
    done += run;
  }
}

// position of group row r inside its slot (SwiGLU groups are stored gate rows first, then up rows)
__device__ __forceinline__ int slot_row(bool swiglu, int r, int nr) { return swiglu ? (r >> 1) + (r & 1) * (nr >> 1) : r; }

}  // namespace
