// Radix-r store-and-forward (Bruck style) routing of per-destination blocks
// with b exchanges batched per synchronisation: reduce-scatter and all-to-all.
//
// Behaviour reproduced (not code):
//   testing/custom_implementations/work_dir/reduce_scatter/tuna_based_outdated/
//       reduce_scatter_radix_block_0_1.cpp:34-299      (reduce-scatter)
//   testing/custom_implementations/work_dir/reduce_scatter/debug/tuna.cpp:9-270  (all-to-all-v)
//
// A block that source s owes destination d has relative index i = (s - d) mod P.
// Written in base r, every non-zero digit z at position x moves the block
// z * r^x ranks towards d; digits are consumed from the least significant one.
// Blocks are not combined on the way (a parked block keeps its identity), so
// the traffic is all-to-all sized; a block whose remaining digits are all
// zero has arrived and is reduced (reduce-scatter) or stored (all-to-all).
// For each digit position the r-1 digit values are exchanged in batches of b;
// a batch ends with a synchronisation (fence), which is the "b-way batched
// sends" knob of the original algorithm.
#include <algorithm>
#include <stdexcept>

#include "algos.h"

namespace chb {

namespace {

// mode 0: reduce into (dbuf, doff) [n elements]; mode 1: store block of source
// s at (dbuf, doff + s*n).
void emit_tuna(Builder& B, int P, int64_t n, int r, int b, int mode, int dbuf, int64_t doff) {
  if (r < 2) r = 2;
  if (P > 2 && r > P - 1) r = P - 1;
  if (b <= 0 || b > P) b = P;
  int w = 0;
  for (int m = P - 1; m > 0; m /= r) ++w;
  // own block
  for (int d = 0; d < P; ++d) {
    if (mode == 0) B.copy(d, dbuf, doff, d, L_IN, (int64_t)d * n, n);
    else B.copy(d, dbuf, doff + (int64_t)d * n, d, L_IN, (int64_t)d * n, n);
  }
  if (P == 1) return;
  // one parking area per digit position: a block that arrives while digit x is
  // processed is parked in area x and read from there when its next non-zero
  // digit is processed, so arrivals never overwrite blocks that still have to leave
  int PARK = B.tmp((int64_t)std::max(1, w) * (P - 1) * n);
  auto park_off = [&](int area, int i) { return ((int64_t)area * (P - 1) + (i - 1)) * n; };
  auto prev_digit_pos = [&](int i, int x) {  // highest non-zero digit position below x
    int pos = -1;
    int64_t q = 1;
    for (int y = 0; y < x; ++y, q *= r)
      if ((i / q) % r != 0) pos = y;
    return pos;
  };
  B.fence();
  int64_t pw = 1;  // r^x
  for (int x = 0; x < w; ++x, pw *= r) {
    std::vector<int> zs;
    for (int z = 1; z < r; ++z)
      if ((int64_t)z * pw <= P - 1) zs.push_back(z);
    for (size_t k0 = 0; k0 < zs.size(); k0 += (size_t)b) {
      size_t k1 = std::min(zs.size(), k0 + (size_t)b);
      for (int me = 0; me < P; ++me) {
        std::vector<Src> finals;
        for (size_t zi = k0; zi < k1; ++zi) {
          int z = zs[zi];
          int from = (int)((me + (int64_t)z * pw) % P);
          for (int i = 1; i < P; ++i) {
            if ((i / pw) % r != z) continue;
            int64_t hi_next = (i / (pw * r)) * (pw * r);  // digits above x
            int d = (int)(((me - hi_next) % P + P) % P);  // destination of this block
            Src s = (i % pw == 0) ? Src{from, L_IN, (int64_t)d * n}
                                  : Src{from, PARK, park_off(prev_digit_pos(i, x), i)};
            if (hi_next == 0) {
              // arrives: d == me
              if (mode == 0) finals.push_back(s);
              else {
                int src_rank = (d + i) % P;
                B.copy(me, dbuf, doff + (int64_t)src_rank * n, s.peer, s.buf, s.off, n);
              }
            } else {
              B.copy(me, PARK, park_off(x, i), s.peer, s.buf, s.off, n);
            }
          }
        }
        if (!finals.empty()) B.reduce(me, dbuf, doff, finals, n, true);
      }
      B.fence();
    }
  }
}

}  // namespace

void emit_rs_tuna(Builder& B, int P, int64_t n, int r, int b, int dbuf, int64_t doff) {
  emit_tuna(B, P, n, r, b, 0, dbuf, doff);
}

Builder gen_rs_tuna(int P, int64_t n, int r, int b) {
  Builder B(P, (int64_t)P * n, n, "reduce_scatter_radix_block");
  emit_tuna(B, P, n, r, b, 0, L_OUT, 0);
  return B;
}

Builder gen_a2a_tuna(int P, int64_t n, int r, int b) {
  Builder B(P, (int64_t)P * n, (int64_t)P * n, "alltoall_tuna");
  emit_tuna(B, P, n, r, b, 1, L_OUT, 0);
  return B;
}

// direct all-to-all: every rank fetches its block from every source
Builder gen_a2a_linear(int P, int64_t n) {
  Builder B(P, (int64_t)P * n, (int64_t)P * n, "alltoall_linear");
  for (int me = 0; me < P; ++me)
    for (int i = 0; i < P; ++i) {
      int s = (me + i) % P;
      B.copy(me, L_OUT, (int64_t)s * n, s, L_IN, (int64_t)me * n, n);
    }
  return B;
}

}  // namespace chb

// ---- all-to-all-v: per-pair element counts (counts[s*P + d] = elements rank s
// owes rank d), blocks packed in destination order in the input and in source
// order in the output, as MPI_Alltoallv with contiguous displacements.  Same
// radix-r / batch-b routing as above (the algorithm the reference's
// store-and-forward reduce-scatter was derived from, debug/tuna.cpp:9-270).
namespace chb {

Builder gen_a2av_tuna(int P, const std::vector<int64_t>& counts, int r, int b) {
  if ((int)counts.size() != P * P) throw std::runtime_error("alltoallv needs a P x P count matrix");
  for (int64_t c : counts) if (c < 0) throw std::runtime_error("alltoallv counts must be >= 0");
  auto cnt = [&](int s, int d) { return counts[(size_t)s * P + d]; };
  std::vector<int64_t> sdis((size_t)P * P), rdis((size_t)P * P);
  int64_t in_e = 0, out_e = 0, maxc = 0;
  for (int s = 0; s < P; ++s) {
    int64_t a = 0;
    for (int d = 0; d < P; ++d) { sdis[(size_t)s * P + d] = a; a += cnt(s, d); maxc = std::max(maxc, cnt(s, d)); }
    in_e = std::max(in_e, a);
  }
  for (int d = 0; d < P; ++d) {
    int64_t a = 0;
    for (int s = 0; s < P; ++s) { rdis[(size_t)d * P + s] = a; a += cnt(s, d); }
    out_e = std::max(out_e, a);
  }
  Builder B(P, std::max<int64_t>(in_e, 1), std::max<int64_t>(out_e, 1), "alltoallv_tuna");
  if (r < 2) r = 2;
  if (P > 2 && r > P - 1) r = P - 1;
  if (b <= 0 || b > P) b = P;
  for (int d = 0; d < P; ++d)
    B.copy(d, L_OUT, rdis[(size_t)d * P + d], d, L_IN, sdis[(size_t)d * P + d], cnt(d, d));
  if (P == 1) return B;
  int w = 0;
  for (int m = P - 1; m > 0; m /= r) ++w;
  const int64_t slot = std::max<int64_t>(maxc, 1);
  int PARK = B.tmp((int64_t)w * (P - 1) * slot);
  auto park_off = [&](int area, int i) { return ((int64_t)area * (P - 1) + (i - 1)) * slot; };
  auto prev_digit_pos = [&](int i, int x) {
    int pos = -1;
    int64_t q = 1;
    for (int y = 0; y < x; ++y, q *= r)
      if ((i / q) % r != 0) pos = y;
    return pos;
  };
  B.fence();
  int64_t pw = 1;
  for (int x = 0; x < w; ++x, pw *= r) {
    std::vector<int> zs;
    for (int z = 1; z < r; ++z)
      if ((int64_t)z * pw <= P - 1) zs.push_back(z);
    for (size_t k0 = 0; k0 < zs.size(); k0 += (size_t)b) {
      size_t k1 = std::min(zs.size(), k0 + (size_t)b);
      for (int me = 0; me < P; ++me)
        for (size_t zi = k0; zi < k1; ++zi) {
          int z = zs[zi];
          int from = (int)((me + (int64_t)z * pw) % P);
          for (int i = 1; i < P; ++i) {
            if ((i / pw) % r != z) continue;
            int64_t hi_next = (i / (pw * r)) * (pw * r);
            int d = (int)(((me - hi_next) % P + P) % P);
            int s = (d + i) % P;                       // origin of this block
            int64_t c = cnt(s, d);
            if (c == 0) continue;
            Src src = (i % pw == 0) ? Src{from, L_IN, sdis[(size_t)s * P + d]}
                                    : Src{from, PARK, park_off(prev_digit_pos(i, x), i)};
            if (hi_next == 0) B.copy(me, L_OUT, rdis[(size_t)d * P + s], src.peer, src.buf, src.off, c);
            else B.copy(me, PARK, park_off(x, i), src.peer, src.buf, src.off, c);
          }
        }
      B.fence();
    }
  }
  return B;
}

}  // namespace chb
