// Shared definitions of the B200 MoE expert-FFN backend: resident tensor
// record, per-device context, the packed weight layout and the work
// descriptors the streaming GEMV kernels consume.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stddef.h>

// ---------------------------------------------------------------------------
// Packed weight layout ("tile stream").
//
// A matrix W[O, I] (O output rows, I = contraction length) is cut into tiles
// of 32 output rows; a tile is cut along I into blocks of 128 columns. One
// block is stored as one contiguous chunk
//     [2048 B of 4-bit codes][scale bytes]
// and the chunks of a tile follow each other in ascending column order, so a
// tile's whole contraction is one linear stream (bulk-copyable without a
// tensor map) and any column range of it is contiguous as well.
//
// Inside the 2048-byte code part the order is the register order of the
// m16n8k16 tensor-core A fragment, so a lane's 128-bit shared-memory load
// yields finished fragments: with lane = g*4+t (g = 0..7, t = 0..3), slot
// j = sub*2+h (sub = 16-row half of the tile, h = row g or g+8) sits at byte
// j*512 + lane*16 and holds four 32-bit words, one per 32-column group. Word
// (j, lane, grp) carries row sub*16+h*8+g, columns grp*32 + 8t + {0..7}, as
// eight 4-bit fields in the order {0,2,4,6,1,3,5,7} (field f at bits 4f..4f+3),
// which lets two mask operations split a word into the (k, k+1) half2 pairs
// the fragment wants. (A group-major order with 32-bit loads and a rolled loop
// over the groups was measured slower: the kernels are bound by the integer
// pipe, so fewer, wider loads win over a smaller instruction footprint.)
//   int4 (fmt 2, 4): a field is the stored offset-binary nibble (value+8).
//   MXFP4 (fmt 7):   the four (k,k+1) pairs A,B,C,D of a word are re-encoded so
//                    that each decodes with shifts and masks straight into
//                    fp16 bit patterns: per 16-bit half, magnitude bits
//                    (e1 e0 m) at 11..9 / 8..6 / 5..3 / 2..0 and sign bits at
//                    15 / 12 / 13 / 14 for A/B/C/D. An fp16 with those three
//                    bits in its exponent/mantissa top is e2m1 * 2^-14.
//
// Scale part, by mode (always four 32-column slots per block; a group size of
// 64 or 128 repeats its scale):
//   SC_ROW   nothing (one f32 per output row lives in a separate array)
//   SC_H16   fp16 [sub][g][h][grp]  (256 B)  int4 scales that are exact in fp16
//   SC_F32   f32  [sub][g][h][grp]  (512 B)  any other int4 scale
//   SC_MX    u8   [sub][g][h][grp]  (128 B)  ue8m0 exponents
// ---------------------------------------------------------------------------
enum ScaleMode { SC_ROW = 0, SC_H16 = 1, SC_F32 = 2, SC_MX = 3 };

#define TILE_ROWS 32
#define BLOCK_K 128
#define CODE_BYTES 2048

__host__ __device__ inline int scale_bytes_of(int mode) {
    return mode == SC_H16 ? 256 : mode == SC_F32 ? 512 : mode == SC_MX ? 128 : 0;
}
__host__ __device__ inline int chunk_bytes_of(int mode) { return CODE_BYTES + scale_bytes_of(mode); }

struct ColiCudaTensor {
    int fmt, I, O, device, gs, ng;
    size_t logical_bytes;     // what coli_cuda_stats reports: container weights + scales
    size_t physical_bytes;    // what is actually allocated on the device
    // raw storage (tensors the packed layout does not cover)
    void *raw_w;              // bytes as uploaded
    void *raw_s;              // f32 scales, or ue8m0 bytes for fmt 7
    // packed storage
    int packed;               // 1: tile-stream layout below is the only copy
    int mode;                 // ScaleMode
    uint8_t *pk;              // tile streams
    float *rowscale;          // SC_ROW only
    // tensor-core path (gemm_tc.cuh): usable for this tensor, and the power of two its
    // fp16 weight terms are pre-multiplied with
    int tc_ok, tc_shift;
};

// One matrix x one pass of rows for the streaming GEMV kernel.
#define SEG_MAX_ROWS 32
struct GemvSeg {
    const uint8_t *w;         // packed tensor base
    const float *rowscale;    // SC_ROW: [O]
    float *out;               // partial sums: out[(kpart*npos + pos0 + r)*O + o]
    int rowid[SEG_MAX_ROWS];  // rows of the B operand this pass multiplies
    int nrows, pos0;
    int O, ntiles, nkb;       // output rows, tiles (O/32), blocks along I (I/128)
    int nkpart, kb_per_part;  // split of the contraction into partial sums
    int task0;                // index of this segment's first task
};

// Control block of one GEMV launch (device memory).
struct GemvCtl {
    int nseg, ntask, npos;
    int tasks_per_seg;   // > 0 when every segment has this many tasks (then seg = task / tasks_per_seg)
};

#define KSTAT_MBAR_TIMEOUT 1

// The status word lives in pinned host memory that the device addresses directly, so the
// host reads it after a stream synchronisation without a copy. Kernels only ever store a
// non-zero code into it (a plain store: no atomics across the bus are needed for that).
__device__ __forceinline__ void kstat_set(int *status, int code) {
    *reinterpret_cast<volatile int *>(status) = code;
    __threadfence_system();
}

// Routing rule of a layer (device-visible mirror of ColiCudaMoeDesc).
struct RouteRule {
    int D, I, E, K;
    int gating, norm_topk;
    float routed_scale, topp;
};
