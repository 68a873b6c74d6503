// aten::_dyn_quant_matmul_4bit for at most 16 rows of activations (decoding): bound by streaming the int4 weights from
// HBM once, and still bit for bit the reference's arithmetic (crates/vkcore/shaders/qmm4.slang:183-247: per block of bs
// values of k an exact integer sum, converted, multiplied by the block's scale and added to the row's float32 sum in
// block order, first block assigning; then times 1 / activation scale, plus bias).
//
// The float32 sum of an output is a chain along k that cannot be cut into partial sums, so the unit of parallel work is
// a group of 8 output columns over all of k, and every compute warp is a little machine of its own: it owns one group
// at a time, streams that group's weights through a private ring of shared-memory slots (lane 0 issues untiled bulk
// copies, one mbarrier per slot), and needs no other warp. With 16 such warps per SM, ~1800 groups in a typical layer
// and a long chain per group (k / 32 steps whose only serial part is one float add), the SMs' latencies are covered
// by the warps' own instruction-level parallelism.
//
// Weights: real nibbles, re-tiled once per packed tensor (tvb_qmm4_decode_prepare; 0.5 byte per weight plus the
// float32 block scales) into records of 512 values of k for 8 columns: [32-k step][column][16 bytes] followed by the
// record's [block][column] scales, so that a warp's read of a step is one contiguous 128 bytes.
// Activations: int8 from PHASE 0 (qmm4_tc.cu's kernel and layout), rearranged once per CTA into MMA fragment order in
// shared memory (one 16-byte read per lane and step, shared by all warps).
// Integer sums: mma.sync.m16n8k32 (s8 x s8 -> s32), the 16 activation rows as the 16-row operand, 8 weight columns as
// the 8-column operand; (q - zero_point) is fed as q plus a constant operand, two MMAs into one accumulator (three for a
// row whose zero point is -128). Every wait is bounded.
#include <cuda.h>

#include <algorithm>

#include "../core/common.h"
#include "numerics.cuh"
#include "ptx.cuh"

namespace tvb {

// PHASE 0 of qmm4_tc.cu: int8 activations [m, k + 64] (the tail holds the two halves of -zero_point), 1 / scale per row.
int qmm4_quantize_rows(cudaStream_t stream, const void* inp, int dtype, int64_t m, int64_t k, int groupwise, int8_t* q, float* recip,
                       int32_t* neg_zp);

namespace {

constexpr int kCols = 8;          // output columns per group (the MMA's 8-column operand)
constexpr int kWarps = 16;        // compute warps per CTA, each on its own group
constexpr int kChunkK = 512;      // values of k per record
constexpr int kChunkSteps = kChunkK / 32;
constexpr int kChunkWeightBytes = kChunkSteps * kCols * 16;  // 2048
constexpr int kExtraCols = 64;    // the activation rows' tail (o1, o2), as written by PHASE 0

struct DecodeParams {
  const uint8_t* prepared;  // [group][chunk] records
  const int8_t* q;          // [m, k + 64]
  const float* recip;       // [m]
  const float* bias;        // [n] or NULL
  void* out;                // [m, n] float32 or bfloat16
  int* status;
  int m, n, k;
  int steps_per_block;      // bs / 32
  int groups;               // n / 8
  int chunks;               // k / 512
  int record_bytes;         // 2048 weight bytes + 8 * (512 / bs) * 4 scale bytes
  int slots;                // records in flight per warp
  int out_bf16;
};

__device__ __forceinline__ void mma_s8_16832(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                             uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Shared-memory loads by 32-bit shared address (kept out of the generic path, whose latency is that of a global load).
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ float2 lds64f(uint32_t addr) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
               "r"(bytes), "r"(bar)
               : "memory");
}

// Four nibbles (v + 8 each, v in [-8, 7]) in the low halves of a word's bytes -> four int8 v: flipping bit 3 gives v
// as a 4-bit two's complement; its sign bit times 0x1E fills the byte's upper half (0xF0) without carrying across bytes.
__device__ __forceinline__ uint32_t nibbles_to_int8(uint32_t low_nibbles) {
  const uint32_t x = low_nibbles ^ 0x08080808u;
  return (x & 0x08080808u) * 0x1Eu + x;
}

// float(i) for |i| < 2^22 without the conversion unit: the bits of 12582912 + i, minus 12582912 (both exact). A block sum is
// at most 512 * 255 * 8 in magnitude.
__device__ __forceinline__ float exact_float(int i) { return __fsub_rn(__int_as_float(i + 0x4B400000), 12582912.0f); }

// SPB: 32-k steps per block (bs / 32). HI: activation rows 8-15 exist (m > 8); without them half of every block's
// arithmetic is dropped.
template <int SPB, bool HI>
__global__ void __launch_bounds__(kWarps * 32, 1) qmm4_decode_kernel(const DecodeParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (ptx::smem_u32(smem_raw) + 127u) & ~127u;
  uint8_t* base_ptr = smem_raw + (base - ptx::smem_u32(smem_raw));
  // [activation fragments: k / 32 steps x 32 lanes x 16 bytes][per warp: slots x record][barriers: warps x slots]
  const int steps = p.k / 32;
  const int frag_bytes = steps * 32 * 16;
  uint4* frags = reinterpret_cast<uint4*>(base_ptr);
  const int ring_bytes = p.slots * p.record_bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(base_ptr + frag_bytes + kWarps * ring_bytes);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + kWarps * p.slots);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;  // g: activation row (and g + 8) / weight column of this lane's fragments; t: its k piece
  const int64_t qstride = p.k + kExtraCols;
  if (threadIdx.x == 0) {
    for (int i = 0; i < kWarps * p.slots; i++) ptx::mbar_init(ptx::smem_u32(bars + i), 1);
    *abort_flag = 0;
    ptx::fence_mbar_init();
  }
  const uint32_t ring = base + frag_bytes + warp * ring_bytes;
  const uint32_t bar0 = ptx::smem_u32(bars + warp * p.slots);
  const int total_warps = gridDim.x * kWarps;
  // (groups dealt out across the CTAs first, so that every SM gets its share of warps with work)
  const int first_grp = warp * gridDim.x + blockIdx.x;
  auto fill_ring = [&](int grp, long long use) {  // lane 0: the first records of a group into the (free) ring
    const uint8_t* src = p.prepared + static_cast<size_t>(grp) * p.chunks * p.record_bytes;
    const int ahead = p.chunks < p.slots ? p.chunks : p.slots;
    for (int c = 0; c < ahead; c++) {
      const int slot = static_cast<int>((use + c) % p.slots);
      ptx::mbar_expect_tx(bar0 + 8 * slot, static_cast<uint32_t>(p.record_bytes));
      bulk_load(ring + slot * p.record_bytes, src + static_cast<size_t>(c) * p.record_bytes, static_cast<uint32_t>(p.record_bytes),
                bar0 + 8 * slot);
    }
  };
  __syncthreads();  // (the barriers are initialised)
  ptx::grid_launch_dependents();  // (the next product's PHASE 0 may be launched; it waits for this kernel before it touches memory)
  // The weights do not depend on the kernel before this one (PHASE 0, which writes q): start their stream, then wait.
  if (lane == 0 && first_grp < p.groups) fill_ring(first_grp, 0);
  ptx::grid_dependency_wait();
  // Activation fragments, once per CTA. A lane's 8 values of k within a step are 8 t ... 8 t + 7; the weights' low nibbles
  // are the even ones, the high nibbles the odd ones, and the MMA's k slots pair them the same way on both operands.
  // (all of a thread's loads are issued before any is used: their latencies overlap instead of adding up)
  constexpr int kBatch = 8;
  for (int e0 = threadIdx.x; e0 < steps * 32; e0 += kBatch * kWarps * 32) {
    uint2 lo[kBatch], hi[kBatch];
#pragma unroll
    for (int i = 0; i < kBatch; i++) {
      const int e = e0 + i * kWarps * 32;
      const int step = e >> 5, ln = e & 31, fg = ln >> 2, ft = ln & 3;
      const int kk = step * 32 + 8 * ft;
      lo[i] = make_uint2(0u, 0u);
      hi[i] = make_uint2(0u, 0u);
      if (e < steps * 32 && fg < p.m) lo[i] = *reinterpret_cast<const uint2*>(p.q + fg * qstride + kk);
      if (e < steps * 32 && fg + 8 < p.m) hi[i] = *reinterpret_cast<const uint2*>(p.q + (fg + 8) * qstride + kk);
    }
#pragma unroll
    for (int i = 0; i < kBatch; i++) {
      const int e = e0 + i * kWarps * 32;
      if (e < steps * 32)
        frags[e] = make_uint4(ptx::prmt(lo[i].x, lo[i].y, 0x6420u),   // row g, even k
                              ptx::prmt(hi[i].x, hi[i].y, 0x6420u),   // row g + 8, even k
                              ptx::prmt(lo[i].x, lo[i].y, 0x7531u),   // row g, odd k
                              ptx::prmt(hi[i].x, hi[i].y, 0x7531u));  // row g + 8, odd k
    }
  }
  // -zero_point, the same for every k: in [-127, 128]. All but 128 fit one int8 operand; a row with 128 (zero point -128)
  // takes a second one holding the 1 that is left over.
  int off_lo = 0, off_hi = 0;
  if (g < p.m) off_lo = p.q[g * qstride + p.k] + p.q[g * qstride + p.k + 32];
  if (g + 8 < p.m) off_hi = p.q[(g + 8) * qstride + p.k] + p.q[(g + 8) * qstride + p.k + 32];
  const uint32_t o1_lo = static_cast<uint8_t>(off_lo > 127 ? 127 : off_lo) * 0x01010101u;
  const uint32_t o1_hi = static_cast<uint8_t>(off_hi > 127 ? 127 : off_hi) * 0x01010101u;
  const uint32_t o2_lo = off_lo > 127 ? 0x01010101u : 0u, o2_hi = off_hi > 127 ? 0x01010101u : 0u;
  const bool second = __any_sync(0xffffffffu, (o2_lo | o2_hi) != 0u);
  __syncthreads();

  long long use = 0;  // records this warp has consumed so far (slot = use % slots, parity from use / slots)
  bool ok = true;
  for (int grp = first_grp; grp < p.groups && ok; grp += total_warps) {
    const uint8_t* src = p.prepared + static_cast<size_t>(grp) * p.chunks * p.record_bytes;
    // fill the ring (the warp has finished reading every slot: see the end of the chunk loop); the first group's
    // records are already on their way
    if (lane == 0 && grp != first_grp) fill_ring(grp, use);
    // sums of (row g, column 2t), (row g, column 2t+1), (row g+8, column 2t), (row g+8, column 2t+1)
    // (-0 is the neutral element of float addition for every addend, signed zeros included: adding the first block to
    // it is the reference's assignment)
    float sum[4] = {-0.0f, -0.0f, -0.0f, -0.0f};
    int carry[4] = {0, 0, 0, 0};  // the integer sum of the block in progress
    for (int c = 0; c < p.chunks && ok; c++, use++) {
      const int slot = static_cast<int>(use % p.slots);
      ok = ptx::mbar_wait(bar0 + 8 * slot, static_cast<uint32_t>((use / p.slots) & 1), abort_flag);
      if (!ok) break;
      const uint32_t rec = ring + slot * p.record_bytes;
      // Four steps at a time, stage by stage (loads, nibble conversion, MMAs into separate accumulators, then the blocks'
      // float arithmetic in order): each stage's instructions are independent of one another, which is what keeps a warp
      // issuing while loads and MMAs are in flight.
      constexpr int kBatch = 4;
#pragma unroll
      for (int st0 = 0; st0 < kChunkSteps; st0 += kBatch) {
        uint4 a[kBatch];
        uint32_t w[kBatch];
#pragma unroll
        for (int i = 0; i < kBatch; i++) {
          a[i] = ptx::lds128(base + ((c * kChunkSteps + st0 + i) * 32 + lane) * 16);
          // this lane's 8 weights of the step: column g, k = 8 t ... 8 t + 7, as 8 nibbles
          w[i] = lds32(rec + ((st0 + i) * kCols + g) * 16 + 4 * t);
        }
        int acc[kBatch][4], acc_o[kBatch][4];
#pragma unroll
        for (int i = 0; i < kBatch; i++) {
          const uint32_t b_even = nibbles_to_int8(w[i] & 0x0f0f0f0fu);
          const uint32_t b_odd = nibbles_to_int8((w[i] >> 4) & 0x0f0f0f0fu);
#pragma unroll
          for (int j = 0; j < 4; j++) acc[i][j] = acc_o[i][j] = 0;
          mma_s8_16832(acc[i], a[i].x, a[i].y, a[i].z, a[i].w, b_even, b_odd);
          mma_s8_16832(acc_o[i], o1_lo, o1_hi, o1_lo, o1_hi, b_even, b_odd);
          if (second) mma_s8_16832(acc_o[i], o2_lo, o2_hi, o2_lo, o2_hi, b_even, b_odd);
        }
#pragma unroll
        for (int i = 0; i < kBatch; i++) {
          const int st = st0 + i;
#pragma unroll
          for (int j = 0; j < 4; j++) carry[j] += acc[i][j] + acc_o[i][j];  // (integer sums: exact in any order)
          if ((st + 1) % SPB == 0) {
            // the block is complete: float(sum) * scale, added in block order
            const int blk_in_chunk = st / SPB;
            const float2 sc = lds64f(rec + kChunkWeightBytes + (blk_in_chunk * kCols + 2 * t) * 4);
            sum[0] = __fadd_rn(sum[0], __fmul_rn(exact_float(carry[0]), sc.x));
            sum[1] = __fadd_rn(sum[1], __fmul_rn(exact_float(carry[1]), sc.y));
            if (HI) {
              sum[2] = __fadd_rn(sum[2], __fmul_rn(exact_float(carry[2]), sc.x));
              sum[3] = __fadd_rn(sum[3], __fmul_rn(exact_float(carry[3]), sc.y));
            }
            carry[0] = carry[1] = carry[2] = carry[3] = 0;
          }
        }
      }
      // the slot is free: bring in the record `slots` further on
      __syncwarp();
      if (lane == 0 && c + p.slots < p.chunks) {
        ptx::mbar_expect_tx(bar0 + 8 * slot, static_cast<uint32_t>(p.record_bytes));
        bulk_load(ring + slot * p.record_bytes, src + static_cast<size_t>(c + p.slots) * p.record_bytes,
                  static_cast<uint32_t>(p.record_bytes), bar0 + 8 * slot);
      }
    }
    if (!ok) break;
    // times 1 / activation scale, plus bias, clamp, store
    const int col = grp * kCols + 2 * t;
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int row = i < 2 ? g : g + 8;
      const int cc = col + (i & 1);
      if (row >= p.m || cc >= p.n) continue;
      float v = __fmul_rn(sum[i], p.recip[row]);
      if (p.bias != nullptr) v = __fadd_rn(v, p.bias[cc]);
      const float hi = p.out_bf16 ? 3.38953139e38f : 3.40282347e38f;
      v = v < -hi ? -hi : v;  // (NaN passes, as in the reference)
      v = hi < v ? hi : v;
      const int64_t o = static_cast<int64_t>(row) * p.n + cc;
      if (p.out_bf16) static_cast<uint16_t*>(p.out)[o] = static_cast<uint16_t>(__float_as_uint(v) >> 16);
      else static_cast<float*>(p.out)[o] = v;
    }
  }
  if (!ok && lane == 0) atomicExch(p.status, 6);
}

// packed (the float-encoded bytes and the scales of aten::_dyn_quant_pack_4bit_weight) -> records
__global__ void qmm4_decode_prepare_kernel(const float* __restrict__ packed, uint8_t* __restrict__ prepared, int n, int k, int bs) {
  const int groups = n / kCols, chunks = k / kChunkK, nblocks = k / bs, blocks_per_chunk = kChunkK / bs;
  const int weight_words = kChunkWeightBytes / 4, scale_words = kCols * blocks_per_chunk;
  const int record_words = weight_words + scale_words;
  const int64_t wcount = static_cast<int64_t>(n) * k / 2;
  const int64_t total = static_cast<int64_t>(groups) * chunks * record_words;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  uint32_t* out = reinterpret_cast<uint32_t*>(prepared);
  for (int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < total; e += stride) {
    const int64_t rec = e / record_words;
    const int r = static_cast<int>(e % record_words);
    const int grp = static_cast<int>(rec / chunks), c = static_cast<int>(rec % chunks);
    if (r < weight_words) {
      // word (step, column cc, piece t): bytes 4 t ... 4 t + 3 of the step's 16 bytes of column grp * 8 + cc
      const int st = r / (kCols * 4), cc = (r / 4) % kCols, t = r % 4;
      const int64_t src = static_cast<int64_t>(grp * kCols + cc) * (k / 2) + (c * kChunkSteps + st) * 16 + 4 * t;
      uint32_t w = 0;
      for (int i = 0; i < 4; i++) w |= (static_cast<uint32_t>(packed[src + i]) & 0xffu) << (8 * i);
      out[e] = w;
    } else {
      const int q = r - weight_words, blk = q / kCols, cc = q % kCols;
      out[e] = __float_as_uint(packed[wcount + static_cast<int64_t>(grp * kCols + cc) * nblocks + c * blocks_per_chunk + blk]);
    }
  }
}

uint64_t align256(uint64_t x) { return (x + 255) & ~uint64_t(255); }

int record_bytes_of(int64_t bs) { return static_cast<int>(kChunkWeightBytes + kCols * (kChunkK / bs) * 4); }

// records in flight per warp, given what the activation fragments leave of the shared memory
int slots_for(int64_t k, int64_t bs) {
  const int64_t frag_bytes = (k / 32) * 32 * 16;
  const int64_t left = 216 * 1024 - frag_bytes;
  const int64_t slots = left / (static_cast<int64_t>(kWarps) * record_bytes_of(bs));
  return static_cast<int>(std::min<int64_t>(slots, 8));
}

}  // namespace
}  // namespace tvb

using namespace tvb;

extern "C" int tvb_qmm4_decode_usable(int64_t m, int64_t n, int64_t k, int64_t bs) {
  // groups of 8 columns; records of 512 values of k made of whole blocks; room for the activation fragments (16 bytes per
  // value of k) and at least two records in flight per warp
  if (m < 1 || m > 16 || n < 8 || n % 8 != 0 || k < kChunkK || k % kChunkK != 0) return 0;
  if (bs < 32 || bs % 32 != 0 || kChunkK % bs != 0) return 0;
  return slots_for(k, bs) >= 2 ? 1 : 0;
}

extern "C" uint64_t tvb_qmm4_decode_prepared_bytes(int64_t n, int64_t k, int64_t bs) {
  return static_cast<uint64_t>(n / kCols) * static_cast<uint64_t>(k / kChunkK) * static_cast<uint64_t>(record_bytes_of(bs));
}

extern "C" int tvb_qmm4_decode_prepare(int device, const float* packed, int64_t n, int64_t k, int64_t bs, void* prepared,
                                       uint64_t prepared_bytes) {
  TVB_REQUIRE(tvb_qmm4_decode_usable(1, n, k, bs) != 0, "tvb_qmm4_decode_prepare: shape not supported by the decode kernel");
  TVB_REQUIRE(packed != nullptr && prepared != nullptr && prepared_bytes >= tvb_qmm4_decode_prepared_bytes(n, k, bs),
              "tvb_qmm4_decode_prepare: NULL pointer or buffer too small");
  TVB_REQUIRE((reinterpret_cast<uintptr_t>(prepared) & 15u) == 0, "tvb_qmm4_decode_prepare: the buffer must be 16-byte aligned");
  cudaStream_t stream;
  if (enter(device, &stream) != 0) return -1;
  const int64_t words = static_cast<int64_t>(tvb_qmm4_decode_prepared_bytes(n, k, bs) / 4);
  const int grid = static_cast<int>(std::min<int64_t>(static_cast<int64_t>(sm_count(device)) * 16, ceil_div(words, 256)));
  qmm4_decode_prepare_kernel<<<grid, 256, 0, stream>>>(packed, static_cast<uint8_t*>(prepared), static_cast<int>(n),
                                                        static_cast<int>(k), static_cast<int>(bs));
  return launched("qmm4_decode_prepare", dim3(grid), dim3(256), 0, stream);
}

extern "C" uint64_t tvb_qmm4_decode_workspace_bytes(int64_t m, int64_t k) {
  return align256(static_cast<uint64_t>(m) * static_cast<uint64_t>(k + kExtraCols)) + 2 * align256(static_cast<uint64_t>(m) * 4);
}

extern "C" int tvb_qmm4_decode(int device, const void* inp, int dtype, const float* packed, int has_bias, const void* prepared,
                               void* out, int64_t m, int64_t n, int64_t k, int64_t bs, void* workspace, uint64_t workspace_bytes) {
  TVB_REQUIRE(dtype == TVB_F32 || dtype == TVB_BF16, "tvb_qmm4_decode: input must be float32 or bfloat16");
  TVB_REQUIRE(m >= 0 && n >= 0, "tvb_qmm4_decode: bad size");
  if (m == 0 || n == 0) return 0;
  TVB_REQUIRE(tvb_qmm4_decode_usable(m, n, k, bs) != 0,
              "tvb_qmm4_decode: needs m <= 16, n a multiple of 8, k a multiple of 512 (up to about 8192), a block size that divides 512");
  TVB_REQUIRE(inp != nullptr && packed != nullptr && prepared != nullptr && out != nullptr, "tvb_qmm4_decode: NULL pointer");
  TVB_REQUIRE((reinterpret_cast<uintptr_t>(prepared) & 15u) == 0, "tvb_qmm4_decode: the prepared weights must be 16-byte aligned");
  TVB_REQUIRE(workspace != nullptr && workspace_bytes >= tvb_qmm4_decode_workspace_bytes(m, k), "tvb_qmm4_decode: workspace too small");
  cudaStream_t stream;
  if (enter(device, &stream) != 0) return -1;
  const uint64_t qbytes = align256(static_cast<uint64_t>(m) * static_cast<uint64_t>(k + kExtraCols));
  const uint64_t rbytes = align256(static_cast<uint64_t>(m) * 4);
  int8_t* q = static_cast<int8_t*>(workspace);
  float* recip = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + qbytes);
  int32_t* neg_zp = reinterpret_cast<int32_t*>(static_cast<uint8_t*>(workspace) + qbytes + rbytes);
  if (qmm4_quantize_rows(stream, inp, dtype, m, k, bs != k ? 1 : 0, q, recip, neg_zp) != 0) return -1;

  DecodeParams p{};
  p.prepared = static_cast<const uint8_t*>(prepared);
  p.q = q;
  p.recip = recip;
  const int64_t wcount = n * k / 2;
  p.bias = has_bias ? packed + wcount + n * (k / bs) : nullptr;
  p.out = out;
  if (status_word(device, &p.status) != 0) return -1;
  p.m = static_cast<int>(m);
  p.n = static_cast<int>(n);
  p.k = static_cast<int>(k);
  p.steps_per_block = static_cast<int>(bs / 32);
  p.groups = static_cast<int>(n / kCols);
  p.chunks = static_cast<int>(k / kChunkK);
  p.record_bytes = record_bytes_of(bs);
  p.slots = slots_for(k, bs);
  p.out_bf16 = dtype == TVB_BF16;
  const int frag_bytes = static_cast<int>(k / 32) * 32 * 16;
  const int smem = frag_bytes + kWarps * p.slots * p.record_bytes + kWarps * p.slots * 8 + 16 + 128;
  void (*kernel)(const DecodeParams) = nullptr;
  int which = 0;
  const bool hi = m > 8;
  switch (p.steps_per_block) {
    case 1: kernel = hi ? qmm4_decode_kernel<1, true> : qmm4_decode_kernel<1, false>; which = 0; break;
    case 2: kernel = hi ? qmm4_decode_kernel<2, true> : qmm4_decode_kernel<2, false>; which = 1; break;
    case 4: kernel = hi ? qmm4_decode_kernel<4, true> : qmm4_decode_kernel<4, false>; which = 2; break;
    case 8: kernel = hi ? qmm4_decode_kernel<8, true> : qmm4_decode_kernel<8, false>; which = 3; break;
    default: kernel = hi ? qmm4_decode_kernel<16, true> : qmm4_decode_kernel<16, false>; which = 4; break;
  }
  which = 2 * which + (hi ? 1 : 0);
  static int configured_smem[64][10] = {};
  if (configured_smem[device & 63][which] < smem) {
    TVB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured_smem[device & 63][which] = smem;
  }
  const int grid = static_cast<int>(std::min<int64_t>(sm_count(device), p.groups));
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kWarps * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // (overlaps PHASE 0: see griddepcontrol.wait in the kernel)
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  TVB_CUDA(cudaLaunchKernelEx(&cfg, kernel, p));
  return launched("qmm4_decode", dim3(grid), dim3(kWarps * 32), smem, stream);
}
