// Block and warp state shared by all kernels of the operator: the per-block header in shared memory, tile
// scheduling, the per-tile camera cull, and the two list phases (per-sample records for the older backward and
// the generic kernels, merged row records for the forward and everything built on it).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "fbev.h"
#include "fbev_device.cuh"

namespace fbev {

constexpr int kMaxWarps = 8;
// narrow channel vectors would put up to 32 cells on a warp; the record lists of that many cells
// do not fit the shared-memory budget, so the rest of the lanes idle in the channel phase
constexpr int kMaxCellsPerWarp = 8;

// Shared-memory header of a block: matrices, feature sizes, visible-camera list.
struct BlockHeader {
  float* P;    // [N][12]
  int* fs;     // [N][2]
  int* vis;    // [N]
  int* nvis;   // [1]
  unsigned char* warp_area;
};

__host__ __device__ inline size_t header_bytes(int N) {
  size_t words = (size_t)N * 12 + (size_t)N * 2 + (size_t)N + 4;
  return (words * 4 + 15) & ~(size_t)15;
}

__device__ __forceinline__ BlockHeader carve(unsigned char* smem, int N) {
  BlockHeader h;
  h.P = reinterpret_cast<float*>(smem);
  h.fs = reinterpret_cast<int*>(h.P + (size_t)N * 12);
  h.vis = h.fs + (size_t)N * 2;
  h.nvis = h.vis + N;
  h.warp_area = smem + header_bytes(N);
  return h;
}

// Per-warp shared area: list lengths of this pass, running totals, then the records.
template <int REC_U4>
__host__ __device__ inline size_t warp_bytes(int CPW, int cap) {
  return 256 + (size_t)CPW * cap * REC_U4 * 16;
}

struct Tile {
  int b, x0, y0, x1, y1;
};

__device__ __forceinline__ Tile tile_of(const Dev& p, int tile) {
  Tile t;
  const int per = p.tiles_x * p.tiles_y;
  t.b = tile / per;
  const int r = tile - t.b * per;
  const int ty = r / p.tiles_x, tx = r - ty * p.tiles_x;
  t.x0 = tx * p.TX;
  t.y0 = p.y0 + ty * p.TY;
  t.x1 = min(t.x0 + p.TX, p.X);
  t.y1 = min(t.y0 + p.TY, p.y1);
  return t;
}

// Tile scheduling.  With a scheduler word (FbevProblem.workspace) the grid is one resident wave of
// blocks and every block draws tiles from an atomic counter, fetching the next index while it works
// on the current one; the last block to leave puts both words back to zero for the next launch.
// Without it, block i owns tile i.
struct TileLoop {
  int it;
  int ntiles;
  int* slot;  // shared int[2]

  __device__ __forceinline__ void begin(const Dev& p, int* shared_slot) {
    it = 0;
    ntiles = p.tiles_x * p.tiles_y * p.B;
    slot = shared_slot;
    if (p.sched != nullptr) {
      if (threadIdx.x == 0) slot[0] = (int)atomicAdd(p.sched, 1u);
      __syncthreads();
    }
  }
  // index of the tile of this iteration, or -1 when the block is done
  __device__ __forceinline__ int current(const Dev& p) {
    const int cur = p.sched != nullptr ? slot[it & 1] : (it == 0 ? (int)blockIdx.x : ntiles);
    if (cur >= ntiles) return -1;
    if (p.sched != nullptr && threadIdx.x == 0) slot[(it + 1) & 1] = (int)atomicAdd(p.sched, 1u);
    return cur;
  }
  __device__ __forceinline__ void advance() {
    __syncthreads();  // everyone is done with this tile's shared state; also publishes the prefetched index
    ++it;
  }
  __device__ __forceinline__ void end(const Dev& p) {
    if (p.sched != nullptr && threadIdx.x == 0) {
      __threadfence();  // this block's draws are performed before it reports itself done
      const unsigned done = atomicAdd(p.sched + 1, 1u);
      if (done == gridDim.x - 1) {
        p.sched[0] = 0u;
        p.sched[1] = 0u;
      }
    }
  }
};

// The two schedules of the kernels whose warps work on groups of CPW cells independently of each other
// (forward, feature-gradient and depth-gradient kernels).
//   counter (default): the block draws whole tiles from the atomic counter (TileLoop) and its warps share out
//     the tile's groups, with a barrier per tile; it balances large problems.
//   static (Dev.static_units: one sample, at most a few units per warp): the unit of work is one group of one
//     tile and warp w of the grid takes units w, w + W, w + 2W, ...  The warps of a block still work on the
//     groups of one tile at about the same time (their texels stay in the SM's L1), but none waits for
//     another: no barrier, no atomic.  Forward on the benchmark shape, where a block sees about two tiles:
//     35.0 against 37.6 us; warps drawing units one by one from a counter gave 37.0 us (the groups of a tile
//     then land on different SMs); with many tiles per block the static order loses 10-17 % to the counter.
// Use: begin(); while ((tile = current(p, g_first, g_step)) >= 0) { groups g_first, g_first + g_step, ... ;
// advance(); } end().  In the static schedule the caller loads the sample's matrices once before the loop
// (tile_visibility on tile 0, by the whole block): the loop itself must not meet a block barrier.
struct UnitLoop {
  TileLoop loop;
  bool stat;
  bool draw;  // static order for a warp's first unit only, further units from the scheduler word (FBEV_EXP_DRAW)
  int unit;   // static order: this warp's current unit

  __device__ __forceinline__ void begin(const Dev& p, int* shared_slot, int warp, int nwarps) {
    stat = p.static_units != 0;
    draw = stat && p.sched != nullptr && (p.exp & FBEV_EXP_DRAW) != 0;
    unit = blockIdx.x * nwarps + warp;
    if (!stat) loop.begin(p, shared_slot);
  }
  // tile of this visit, or -1 when done; the caller handles groups g_first, g_first + g_step, ... of it
  __device__ __forceinline__ int current(const Dev& p, int ngroups, int warp, int nwarps, int& g_first, int& g_step) {
    if (stat) {
      if (unit >= p.tiles_x * p.tiles_y * p.B * ngroups) return -1;
      const int tile = unit / ngroups;
      g_first = unit - tile * ngroups;
      g_step = ngroups;  // one group per visit
      return tile;
    }
    g_first = warp;
    g_step = nwarps;
    return loop.current(p);
  }
  __device__ __forceinline__ void advance(const Dev& p, int nwarps) {
    if (draw) {
      // the first round went out in the static order (neighbouring warps on neighbouring groups); what is left is
      // handed out one unit at a time to whichever warp is free, which evens out the unequal cost of the units
      unsigned u = 0;
      if ((threadIdx.x & 31) == 0) u = atomicAdd(p.sched, 1u);
      u = __shfl_sync(kFull, u, 0);
      unit = (int)(gridDim.x * nwarps + u);
    } else if (stat) {
      unit += gridDim.x * nwarps;
    } else {
      loop.advance();
    }
  }
  __device__ __forceinline__ void end(const Dev& p, int nwarps) {
    if (draw) {
      if ((threadIdx.x & 31) == 0) {
        __threadfence();
        const unsigned done = atomicAdd(p.sched + 1, 1u);  // warps that have left
        if (done == gridDim.x * nwarps - 1) {
          p.sched[0] = 0u;
          p.sched[1] = 0u;
        }
      }
    } else if (!stat) {
      loop.end(p);
    }
  }
};

// Loads matrices and feature sizes of the tile's sample (when it differs from the one already in
// shared memory) and builds the list of cameras that may see the tile.  Ends with a block barrier.
__device__ __forceinline__ void block_prologue(const Dev& p, const Tile& t, const BlockHeader& h, const float vs[3],
                                               const float vmin[3], int image_h, int image_w, int& loaded_b) {
  const int tid = threadIdx.x, nt = blockDim.x;
  if (loaded_b != t.b) {
    for (int i = tid; i < p.N * 12; i += nt) {
      const int n = i / 12, k = i - n * 12;
      h.P[i] = __ldg(p.proj + ((size_t)t.b * p.N + n) * p.pstride + k);
    }
    for (int i = tid; i < p.N * 2; i += nt) h.fs[i] = __ldg(p.fsize + (size_t)t.b * p.N * 2 + i);
    loaded_b = t.b;
  }
  __syncthreads();
  if (tid < 32) {
    const float bx0 = centre(t.x0, vs[0], vmin[0]), bx1 = centre(t.x1 - 1, vs[0], vmin[0]);
    const float by0 = centre(t.y0, vs[1], vmin[1]), by1 = centre(t.y1 - 1, vs[1], vmin[1]);
    const float bz0 = centre(0, vs[2], vmin[2]), bz1 = centre(p.Z - 1, vs[2], vmin[2]);
    int base = 0;
    for (int n0 = 0; n0 < p.N; n0 += 32) {
      const int n = n0 + tid;
      bool see = false;
      if (n < p.N) {
        const int fh = h.fs[n * 2], fw = h.fs[n * 2 + 1];
        const bool ok = fh > 0 && fw > 0 && (long long)fh * fw <= (long long)p.H * p.W;
        if (!ok) {
          if (p.status != nullptr) atomicOr(p.status, (int)FBEV_DEV_BAD_FEATURE_SIZE);
        } else {
          see = camera_may_see(p, h.P + n * 12, bx0, bx1, by0, by1, bz0, bz1, image_h, image_w);
        }
      }
      const unsigned m = __ballot_sync(kFull, see);
      if (see) h.vis[base + __popc(m & ((1u << tid) - 1u))] = n;
      base += __popc(m);
    }
    if (tid == 0) *h.nvis = base;
  }
  __syncthreads();
}

// Bit mask of the cameras (up to 32) that may see a box of cells [t.x0, t.x1) x [t.y0, t.y1) of sample t.b, whose
// matrices are in shared memory; evaluated by every warp for itself, lane n for camera n.  A camera whose
// feature_size entry is unusable (non-positive, larger than the tensor, or beyond what 32-bit chunk indices
// address) is left out and reported in the status word.
__device__ __forceinline__ unsigned box_visibility(const Dev& p, const Tile& t, const BlockHeader& h, const float vs[3],
                                                   const float vmin[3], int image_h, int image_w) {
  const int lane = threadIdx.x & 31;
  bool see = false;
  if (lane < p.N) {
    const int fh = h.fs[lane * 2], fw = h.fs[lane * 2 + 1];
    bool ok = fh > 0 && fw > 0 && (long long)fh * fw <= (long long)p.H * p.W;
    if (ok && p.cpt > 0)  // 32-bit chunk indices into the feature tensor, 32-bit element indices into the depth tensor
      ok = (unsigned long long)((size_t)t.b * p.N + lane + 1) * (unsigned long long)fh * fw * (unsigned)max(p.cpt, p.D) < (1ull << 32);
    if (ok) {
      const float bx0 = centre(t.x0, vs[0], vmin[0]), bx1 = centre(t.x1 - 1, vs[0], vmin[0]);
      const float by0 = centre(t.y0, vs[1], vmin[1]), by1 = centre(t.y1 - 1, vs[1], vmin[1]);
      const float bz0 = centre(0, vs[2], vmin[2]), bz1 = centre(p.Z - 1, vs[2], vmin[2]);
      see = camera_may_see(p, h.P + lane * 12, bx0, bx1, by0, by1, bz0, bz1, image_h, image_w);
    } else if (p.status != nullptr && threadIdx.x < 32) {
      atomicOr(p.status, (int)FBEV_DEV_BAD_FEATURE_SIZE);
    }
  }
  return __ballot_sync(kFull, see);
}

// Forward-kernel prologue for up to 32 cameras.  The matrices are (re)loaded only when the tile
// belongs to another sample than the one in shared memory (block barriers then); the camera cull is
// evaluated by every warp for itself and returned as a bit mask, so the steady state has no barrier.
__device__ __forceinline__ unsigned tile_visibility(const Dev& p, const Tile& t, const BlockHeader& h,
                                                    const float vs[3], const float vmin[3], int image_h, int image_w,
                                                    int& loaded_b) {
  if (loaded_b != t.b) {  // uniform over the block
    __syncthreads();      // nobody still reads the matrices of the sample before
    for (int i = threadIdx.x; i < p.N * 12; i += blockDim.x) {
      const int n = i / 12, k = i - n * 12;
      h.P[i] = __ldg(p.proj + ((size_t)t.b * p.N + n) * p.pstride + k);
    }
    for (int i = threadIdx.x; i < p.N * 2; i += blockDim.x) h.fs[i] = __ldg(p.fsize + (size_t)t.b * p.N * 2 + i);
    loaded_b = t.b;
    __syncthreads();
  }
  return box_visibility(p, t, h, vs, vmin, image_h, image_w);
}

// List phase for one group of cells and one pass over candidates [r0, r1) of
// every cell (candidate r = visible-camera index * Z + z).
//   t0      first tile-linear cell of the group; cell = t0 + c, c < CPW
//   sLen    [CPW] list lengths produced by this pass
//   recs    [CPW][cap] records of REC_U4 uint4 each:
//             [0] bilinear weights w00 w01 w10 w11 (forward: already times the depth weight)
//             [1] texel index of (v0,u0) within the whole feature tensor, u1-u0, (v1-v0)*fw, depth bin
//             [2] backward only: depth weight, d/dmean, d/dsigma, texel-local depth row (unused)
template <typename T, bool BWD, bool COUNT_ONLY>
__device__ __forceinline__ void list_phase(const Dev& p, const Tile& t, const BlockHeader& h, int nvis, int t0,
                                           int r0, int r1, const float vs[3], const float vmin[3], int image_h,
                                           int image_w, int* sLen, uint4* recs, int lane) {
  constexpr int REC_U4 = BWD ? 3 : 2;
  const int per = r1 - r0;
  const int total = p.CPW * per;
  const int tile_cells = p.TX * p.TY;
  if (lane < p.CPW) sLen[lane] = 0;
  __syncwarp();
  for (int base = 0; base < total; base += 32) {
    const int q = base + lane;
    bool ok = false;
    int cl = 0;
    Sample s;
    size_t tex00 = 0;
    int fw = 0;
    if (q < total) {
      cl = q / per;
      const int r = r0 + (q - cl * per);
      const int ci = r / p.Z, z = r - ci * p.Z;
      const int tc = t0 + cl;
      const int ly = tc / p.TX, lx = tc - ly * p.TX;
      const int x = t.x0 + lx, y = t.y0 + ly;
      if (tc < tile_cells && x < t.x1 && y < t.y1 && ci < nvis) {
        const int n = h.vis[ci];
        const int fh = h.fs[n * 2];
        fw = h.fs[n * 2 + 1];
        const float vx = centre(x, vs[0], vmin[0]), vy = centre(y, vs[1], vmin[1]), vz = centre(z, vs[2], vmin[2]);
        if (geometry(h.P + n * 12, vx, vy, vz, image_h, image_w, fh, fw, p.eps, s)) {
          const size_t texbase = ((size_t)t.b * p.N + n) * (size_t)fh * fw;
          ok = depth_weight<T, BWD>(p, texbase, fw, s);
          tex00 = texbase + (size_t)s.v0 * fw + s.u0;
        }
      }
    }
    const unsigned vm = __ballot_sync(kFull, ok);
    // lanes [lo, hi) of this sweep hold candidates of cell cl
    const int lo = min(max(cl * per - base, 0), 31);
    const int hi = min(max((cl + 1) * per - base, 0), 32);
    const unsigned seg = (hi >= 32 ? kFull : ((1u << hi) - 1u)) & ~((1u << lo) - 1u);
    const int before = sLen[cl];
    __syncwarp();
    if (!COUNT_ONLY && ok) {
      const int pos = before + __popc(vm & seg & ((1u << lane) - 1u));
      uint4* rec = recs + ((size_t)cl * p.cap + pos) * REC_U4;
      if (BWD) {
        rec[0] = make_uint4(__float_as_uint(s.w00), __float_as_uint(s.w01), __float_as_uint(s.w10),
                            __float_as_uint(s.w11));
        rec[2] = make_uint4(__float_as_uint(s.wgt), __float_as_uint(s.dmean), __float_as_uint(s.dsigma), 0u);
      } else {
        rec[0] = make_uint4(__float_as_uint(s.w00 * s.wgt), __float_as_uint(s.w01 * s.wgt),
                            __float_as_uint(s.w10 * s.wgt), __float_as_uint(s.w11 * s.wgt));
      }
      rec[1] = make_uint4((uint32_t)tex00, (uint32_t)(s.u1 - s.u0), (uint32_t)((s.v1 - s.v0) * fw), (uint32_t)s.k);
    }
    if (q < total && lane == lo) sLen[cl] = before + __popc(vm & seg);
    __syncwarp();
  }
}

// One 16-byte chunk of channels of the output (or of the upstream gradient): element type T, or
// float32 when a 16-bit operator was asked for a float32 output.  `chunk` counts T-sized chunks.
template <typename T>
__device__ __forceinline__ void store_chunk(void* base, int as_f32, size_t chunk, const float* v) {
  constexpr int E = Chunk<T>::E;
  if (E == 8 && as_f32) {
    float4* o = reinterpret_cast<float4*>(base) + chunk * 2;
    o[0] = make_float4(v[0], v[1], v[2], v[3]);
    o[1] = make_float4(v[4], v[5], v[6], v[7]);
  } else {
    reinterpret_cast<uint4*>(base)[chunk] = Chunk<T>::pack(v);
  }
}
// The same chunk stored once to a multicast address: the NVSwitch delivers it to the buffer of every GPU bound to
// the multicast object, this one included (multimem.st; a plain store instruction, nothing is loaded or reduced).
__device__ __forceinline__ void multicast_store16(void* addr, float a, float b, float c, float d) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}
template <typename T>
__device__ __forceinline__ void store_chunk_multicast(void* base, int as_f32, size_t chunk, const float* v) {
  constexpr int E = Chunk<T>::E;
  if (E == 8 && as_f32) {
    float4* o = reinterpret_cast<float4*>(base) + chunk * 2;
    multicast_store16(o, v[0], v[1], v[2], v[3]);
    multicast_store16(o + 1, v[4], v[5], v[6], v[7]);
  } else {
    const uint4 q = Chunk<T>::pack(v);  // any 16 bytes travel as four 32-bit words
    multicast_store16(reinterpret_cast<uint4*>(base) + chunk, __uint_as_float(q.x), __uint_as_float(q.y),
                      __uint_as_float(q.z), __uint_as_float(q.w));
  }
}

template <typename T>
__device__ __forceinline__ void load_chunk(const void* base, int as_f32, size_t chunk, float* v) {
  constexpr int E = Chunk<T>::E;
  if (E == 8 && as_f32) {
    const float4* g = reinterpret_cast<const float4*>(base) + chunk * 2;
    const float4 a = __ldg(g), b = __ldg(g + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
    Chunk<T>::unpack(ldg16(reinterpret_cast<const uint4*>(base) + chunk), v);
  }
}

// exact q / d for 0 <= q < 2^21, given inv = 1.0f / d
__device__ __forceinline__ int fast_div(int q, float inv) { return __float2int_rz((__int2float_rn(q) + 0.5f) * inv); }

// Per-warp shared area of the forward kernel: record-list lengths and sample counts, then per cell
// a list of row records (one padding slot per cell keeps the cells' lists on different banks).
__host__ __device__ inline int row_stride(int cap) { return 2 * cap + 1; }
__host__ __device__ inline size_t fwd_warp_bytes(int CPW, int cap) { return 256 + (size_t)CPW * row_stride(cap) * 16; }

// Per-warp shared area of the kernels that also keep every accepted sample (depth gradient, training forward):
// list lengths, sample counts, sample-record counts, the row records, then three 16-byte words per sample.
__host__ __device__ inline size_t depth_warp_bytes(int CPW, int cap) {
  return 512 + (size_t)CPW * row_stride(cap) * 16 + (size_t)CPW * cap * 48;
}

// Lists saved by a training forward for the backward.  The depth-gradient kernel needs exactly what the forward's
// list phase produces, per group of cells and pass: the row records and the sample records.  Rebuilding them costs
// the backward more than everything else it does, so a forward that knows a backward will follow writes them out:
//   saved[0]                      {cursor: 16-byte units handed out so far, plan key, -, -}
//   saved[1 + e]                  directory entry of (unit, pass) e, 16 bytes: the offset of the pass's block in
//                                 16-byte units from saved (kSavedMissing when the data area was full), and the
//                                 cells' list lengths (6 bits each) and sample counts (5 bits each), see pack_counts
//   block                         the cells' row records back to back, then the cells' sample records back to back
// A unit is one group of cells of one tile (tile * groups + group), the same in both kernels as long as both use
// the same tiling and lane layout, which the plan key vouches for.  A block that did not fit is simply rebuilt.
// The directory entry carries the counts so that a reader needs one round trip to memory for them and one for all
// of the block's words, which it requests together.
constexpr unsigned kSavedMissing = 0xffffffffu;

__device__ __forceinline__ uint4* saved_dir_entry(const Dev& p, unsigned unit, int pass) {
  return p.saved + 1 + ((size_t)(p.saved_unit0 + unit) * p.saved_passes + pass);
}

// Up to eight cells with at most 33 records and 16 samples each per pass: 48 bits of lengths (y and the low half of
// z) and 40 bits of counts (w and the high half of z).
__device__ __forceinline__ void pack_counts(const int* sLen, const int* sSmp, int CPW, unsigned& y, unsigned& z, unsigned& w) {
  y = z = w = 0u;
  unsigned long long len = 0, cnt = 0;
  for (int c = 0; c < CPW; ++c) {
    len |= (unsigned long long)(unsigned)sLen[c] << (6 * c);  // <= 33 < 64
    cnt |= (unsigned long long)(unsigned)sSmp[c] << (5 * c);  // <= 16 < 32
  }
  y = (unsigned)len;
  z = (unsigned)(len >> 32) | ((unsigned)(cnt >> 32) << 16);
  w = (unsigned)cnt;
}
__device__ __forceinline__ int saved_len(const uint4& e, int c) {
  const unsigned long long len = (unsigned long long)e.y | ((unsigned long long)(e.z & 0xffffu) << 32);
  return (int)((len >> (6 * c)) & 63u);
}
__device__ __forceinline__ int saved_cnt(const uint4& e, int c) {
  const unsigned long long cnt = (unsigned long long)e.w | ((unsigned long long)(e.z >> 16) << 32);
  return (int)((cnt >> (5 * c)) & 31u);
}

// Writes this warp's lists of one pass (after row_list_phase with SAMPLES) to the saved state.
__device__ __forceinline__ void save_pass(const Dev& p, unsigned unit, int pass, const int* sLen, const int* sSmp,
                                          const uint4* recs, const uint4* samp, int lane) {
  const int rstride = row_stride(p.cap);
  int nrec = 0, nsmp = 0;
  for (int c = 0; c < p.CPW; ++c) {
    nrec += sLen[c];
    nsmp += sSmp[c];
  }
  const unsigned need = (unsigned)nrec + 3u * (unsigned)nsmp;
  const unsigned data0 = 1u + p.saved_dir;
  unsigned off = 0;
  if (lane == 0) off = atomicAdd(reinterpret_cast<unsigned*>(p.saved), need);
  off = __shfl_sync(kFull, off, 0);
  const bool fits = (unsigned long long)off + need <= (unsigned long long)p.saved_cap;
  if (lane == 0) {
    unsigned y, z, w;
    pack_counts(sLen, sSmp, p.CPW, y, z, w);
    *saved_dir_entry(p, unit, pass) = make_uint4(fits ? data0 + off : kSavedMissing, y, z, w);
    if (!fits) reinterpret_cast<unsigned*>(p.saved)[2] = 1u;  // the state is incomplete: the backward rebuilds
  }
  if (!fits) return;
  uint4* dst = p.saved + data0 + off;
  unsigned at = 0;
  for (int c = 0; c < p.CPW; ++c) {
    const int n = sLen[c];
    for (int i = lane; i < n; i += 32) dst[at + i] = recs[(size_t)c * rstride + i];
    at += (unsigned)n;
  }
  for (int c = 0; c < p.CPW; ++c) {
    const int n = 3 * sSmp[c];
    for (int i = lane; i < n; i += 32) dst[at + i] = samp[(size_t)c * p.cap * 3 + i];
    at += (unsigned)n;
  }
}

// True when the saved state at p.saved was written completely, in this launch's layout.  Uniform over the grid.
__device__ __forceinline__ bool saved_usable(const Dev& p) {
  if (p.saved == nullptr) return false;
  const volatile unsigned* head = reinterpret_cast<const volatile unsigned*>(p.saved);  // written by the forward kernel
  return head[1] == p.saved_key && head[2] == 0u;
}

// Reads the lists of one pass back into the warp's shared area; the counterpart of row_list_phase with SAMPLES.
// Adds the pass's sample counts to sCnt, as the list phase does.  All words of the block are requested together
// (four loads in flight per lane), so the pass costs two round trips to memory: the directory entry, then the
// block.  sOff: 2 x (kMaxCellsPerWarp + 1) ints of the warp's shared area for the cells' start offsets.
__device__ __forceinline__ void load_pass(const Dev& p, unsigned unit, int pass, int* sLen, int* sCnt, int* sSmp,
                                          int* sOff, uint4* recs, uint4* samp, int lane) {
  const uint4 e = __ldg(saved_dir_entry(p, unit, pass));
  const uint4* blk = p.saved + e.x;
  const int rstride = row_stride(p.cap);
  // exclusive prefix sums of the cells' record counts and sample words, by the first lanes
  const int l = lane < p.CPW ? saved_len(e, lane) : 0, m = lane < p.CPW ? saved_cnt(e, lane) : 0;
  int pl = l, pm = 3 * m;
#pragma unroll
  for (int d = 1; d < kMaxCellsPerWarp; d <<= 1) {
    const int a = __shfl_up_sync(kFull, pl, d), b = __shfl_up_sync(kFull, pm, d);
    if (lane >= d) {
      pl += a;
      pm += b;
    }
  }
  if (lane < kMaxCellsPerWarp) {
    sOff[lane + 1] = pl;
    sOff[kMaxCellsPerWarp + 1 + lane + 1] = pm;
    if (lane == 0) sOff[0] = sOff[kMaxCellsPerWarp + 1] = 0;
  }
  if (lane < p.CPW) {
    sLen[lane] = l;
    sSmp[lane] = m;
    sCnt[lane] += m;
  }
  __syncwarp();
  const int* rec0 = sOff;
  const int* smp0 = sOff + kMaxCellsPerWarp + 1;
  const int nrec = rec0[kMaxCellsPerWarp], total = nrec + smp0[kMaxCellsPerWarp];
  constexpr int U = 4;
  for (int base = 0; base < total; base += 32 * U) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = base + u * 32 + lane;
      if (i < total) v[u] = __ldg(blk + i);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = base + u * 32 + lane;
      if (i >= total) continue;
      const bool is_rec = i < nrec;
      const int* start = is_rec ? rec0 : smp0;
      const int j = is_rec ? i : i - nrec;
      int c = 0;
#pragma unroll
      for (int k = 1; k < kMaxCellsPerWarp; ++k) c += j >= start[k] ? 1 : 0;
      const int off = j - start[c];
      if (is_rec) {
        v[u].x -= p.saved_sub_rec;  // chunk index of the record's texel, counted from the first sample of this launch
        recs[(size_t)c * rstride + off] = v[u];
      } else {
        if (off % 3 == 1) v[u].x -= p.saved_sub_dep;  // second word of a sample: its depth element index
        samp[(size_t)c * p.cap * 3 + off] = v[u];
      }
    }
  }
  __syncwarp();
}

// List phase of the forward kernel.  As list_phase() it evaluates one candidate per lane, but it
// emits ROW records instead of samples.  A sample touches two feature rows (v0 and v1) at the
// columns (u0, u1); the z samples of one (cell, camera) are neighbouring lanes and mostly fall on
// the same or on adjacent rows, so
//   * neighbouring accepted lanes with the same (cell, camera, texel (v0,u0), u1-u0) form a run whose
//     weights are summed with a segmented warp scan, and
//   * the v1 part of a run is merged with the v0 part of the run before it when that one sits
//     exactly one row further down (the usual order: v decreases as z grows).
// Every run then emits at most two records {texel of (row, u0), u1-u0, weight of u0, weight of u1},
// already multiplied by the depth weight.  The channel phase reads two texels per record instead of
// four per sample, which is some 2.5 to 5 times fewer gathers for the benchmark shapes.  Runs do not
// extend across the 32 candidates of one sweep; that only costs merges, never correctness.
// SAMPLES (depth-gradient kernel): every accepted sample is also kept, per cell, as three uint4
//   [0] bilinear weights w00 w01 w10 w11
//   [1] element index of depth[(v0,u0)][0], element distance to u1, to v1, depth bin (or -1)
//   [2] positions of the row records holding its v0 and its v1 texels (low / high 16 bits), depth
//       weight, d weight / d mean, d weight / d sigma
// in `samp` ([CPW][cap] records), counted in sSmp.
template <typename T, bool WRITE = true, bool SAMPLES = false>
__device__ __forceinline__ void row_list_phase(const Dev& p, const Tile& t, const BlockHeader& h, unsigned vis, unsigned cpt, int t0, int r0,
                                               int r1, const float vs[3], const float vmin[3], int image_h,
                                               int image_w, int* sLen, int* sCnt, uint4* recs, int lane,
                                               uint4* samp = nullptr, int* sSmp = nullptr) {
  const int per = r1 - r0;
  const int total = p.CPW * per;
  const int tile_cells = p.TX * p.TY;
  const int rstride = row_stride(p.cap);
  const float inv_per = 1.0f / (float)per, inv_z = 1.0f / (float)p.Z, inv_tx = 1.0f / (float)p.TX;
  const int z_shift = (p.Z & (p.Z - 1)) == 0 ? 31 - __clz(p.Z) : -1;
  const int row0 = t0 / p.TX;
  const bool one_row = (t0 + p.CPW - 1) / p.TX == row0;  // all cells of the group in one row of the tile
  const unsigned lt = (1u << lane) - 1u;
  // camera of the ci-th set bit of vis, as a byte table in the unused part of sLen (cells use entries 0..7)
  unsigned char* visl = reinterpret_cast<unsigned char*>(sLen + kMaxCellsPerWarp);
  if ((vis >> lane) & 1u) visl[__popc(vis & lt)] = (unsigned char)lane;
  __syncwarp();
  for (int base = 0; base < total; base += 32) {
    const int q = base + lane;
    bool ok = false;
    int cl = 0;
    unsigned tex = 0, kk = 0;
    int fw = 0;
    float A0 = 0.0f, A1 = 0.0f, B0 = 0.0f, B1 = 0.0f;
    Sample s;
    unsigned dep00 = 0;
    if (q < total) {
      cl = fast_div(q, inv_per);
      const int r = r0 + (q - cl * per);
      // camera and height bin: a shift and a mask when Z is a power of two
      const int ci = z_shift >= 0 ? (r >> z_shift) : fast_div(r, inv_z), z = r - ci * p.Z;
      const int tc = t0 + cl;
      // row and column of the cell inside the tile: the group's own row when it lies within one
      const int ly = one_row ? row0 : fast_div(tc, inv_tx), lx = tc - ly * p.TX;
      const int x = t.x0 + lx, y = t.y0 + ly;
      if (tc < tile_cells && x < t.x1 && y < t.y1) {
        const int n = visl[ci];  // ci-th visible camera
        const int fh = h.fs[n * 2];
        fw = h.fs[n * 2 + 1];
        const float vx = centre(x, vs[0], vmin[0]), vy = centre(y, vs[1], vmin[1]), vz = centre(z, vs[2], vmin[2]);
        if (geometry(h.P + n * 12, vx, vy, vz, image_h, image_w, fh, fw, p.eps, s)) {
          const unsigned texbase = (unsigned)(t.b * p.N + n) * (unsigned)(fh * fw);  // below 2^32 / cpt (box_visibility)
          ok = depth_weight<T, SAMPLES, unsigned>(p, texbase, fw, s);
          if (ok) {
            tex = texbase + (unsigned)(s.v0 * fw + s.u0);
            dep00 = tex * (unsigned)p.D;
            const unsigned du = (unsigned)(s.u1 - s.u0), dvf = (unsigned)(s.v1 - s.v0);
            kk = (unsigned)cl | ((unsigned)ci << 4) | (du << 28) | (dvf << 29) | (1u << 31);
            A0 = s.w00 * s.wgt;
            A1 = s.w10 * s.wgt;
            B0 = s.w01 * s.wgt;
            B1 = s.w11 * s.wgt;
            if (!dvf) {  // last feature row: v1 == v0, both parts land on the same texels
              A0 += B0;
              A1 += B1;
              B0 = B1 = 0.0f;
            }
          }
        }
      }
    }
    const unsigned okm = __ballot_sync(kFull, ok);
    // same run as the lane before?
    const unsigned ptex1 = __shfl_up_sync(kFull, tex, 1), pkk1 = __shfl_up_sync(kFull, kk, 1);
    const bool sap = ok && lane > 0 && pkk1 == kk && ptex1 == tex;
    const unsigned sapm = __ballot_sync(kFull, sap);
    const unsigned headm = okm & ~sapm;
    const int rs = 31 - __clz((int)(headm & (lt | (1u << lane))));  // first lane of my run (ok lanes only)
    // segmented inclusive sums over the run
    for (int d = 1; d < 32 && d < p.Z; d <<= 1) {
      const float a0 = __shfl_up_sync(kFull, A0, d), a1 = __shfl_up_sync(kFull, A1, d);
      const float b0 = __shfl_up_sync(kFull, B0, d), b1 = __shfl_up_sync(kFull, B1, d);
      if (ok && lane - d >= rs) {
        A0 += a0;
        A1 += a1;
        B0 += b0;
        B1 += b1;
      }
    }
    const bool tail = ok && (lane == 31 || !((sapm >> (lane + 1)) & 1u));
    // the run before mine ends at lane rs - 1; its tail lane holds its totals
    const int pl = (rs - 1) & 31;
    const unsigned ptex = __shfl_sync(kFull, tex, pl), pkk = __shfl_sync(kFull, kk, pl);
    const float pA0 = __shfl_sync(kFull, A0, pl), pA1 = __shfl_sync(kFull, A1, pl);
    const unsigned ntex = __shfl_down_sync(kFull, tex, 1), nkk = __shfl_down_sync(kFull, kk, 1);
    const unsigned colmask = 0x1fffffffu;  // cell, camera and u1-u0 must agree; not the v1-v0 bit
    const bool has_b = (kk >> 29) & 1u;
    // my v1 part meets the v0 part of the run before me, one row further down
    const bool absorb_prev = tail && has_b && rs > 0 && ((okm >> pl) & 1u) && ((pkk ^ kk) & colmask) == 0 &&
                             ptex == tex + (unsigned)fw;
    // my v0 part is taken by the run after me under the same rule
    const bool given_to_next = tail && lane < 31 && ((okm >> ((lane + 1) & 31)) & 1u) && ((nkk ^ kk) & colmask) == 0 &&
                               ((nkk >> 29) & 1u) && tex == ntex + (unsigned)fw;
    const bool emit_a = tail && !given_to_next;
    const bool emit_b = tail && has_b;
    const unsigned m1 = __ballot_sync(kFull, emit_a || emit_b), m2 = __ballot_sync(kFull, emit_a && emit_b);
    // lanes [lo, hi) of this sweep hold candidates of cell cl
    const int lo = min(max(cl * per - base, 0), 31);
    const int hi = min(max((cl + 1) * per - base, 0), 32);
    const unsigned seg = (hi >= 32 ? kFull : ((1u << hi) - 1u)) & ~((1u << lo) - 1u);
    const int before = sLen[cl];
    __syncwarp();
    const int pos0 = before + __popc(m1 & seg & lt) + __popc(m2 & seg & lt);
    const int pos_a = emit_a ? pos0 : -1;                    // tail lanes: where the run's records go
    const int pos_b = emit_b ? pos0 + (emit_a ? 1 : 0) : -1;
    if (WRITE && tail) {
      uint4* rec = recs + (size_t)cl * rstride;
      const unsigned du = (kk >> 28) & 1u;
      // chunk index of texel (row, u0), chunk distance to (row, u1), weights
      if (emit_a) rec[pos_a] = make_uint4(tex * cpt, du * cpt, __float_as_uint(A0), __float_as_uint(A1));
      if (emit_b)
        rec[pos_b] = make_uint4((tex + (unsigned)fw) * cpt, du * cpt, __float_as_uint(B0 + (absorb_prev ? pA0 : 0.0f)),
                                __float_as_uint(B1 + (absorb_prev ? pA1 : 0.0f)));
    }
    if (SAMPLES) {
      // every sample learns which records hold its texels: its run's tail lane knows
      const unsigned tailm = __ballot_sync(kFull, tail);
      const unsigned ahead = tailm >> lane;                  // bit 0: me
      const int tl = ahead ? lane + __ffs((int)ahead) - 1 : lane;
      const int run_a = __shfl_sync(kFull, pos_a, tl), run_b = __shfl_sync(kFull, pos_b, tl);
      // a run whose v0 part was taken over by the next run finds it in that run's v1 record
      const unsigned after = tl < 31 ? tailm >> (tl + 1) : 0u;
      const int ntl = after ? tl + 1 + __ffs((int)after) - 1 : tl;
      const int next_b = __shfl_sync(kFull, pos_b, ntl);
      if (ok) {
        const int my_a = run_a >= 0 ? run_a : next_b;
        const int my_b = has_b ? run_b : my_a;               // v1 == v0: both parts sit in the v0 record
        const int spos = sSmp[cl] + __popc(okm & seg & lt);
        uint4* sr = samp + ((size_t)cl * p.cap + spos) * 3;
        const unsigned du = (kk >> 28) & 1u;
        sr[0] = make_uint4(__float_as_uint(s.w00), __float_as_uint(s.w01), __float_as_uint(s.w10), __float_as_uint(s.w11));
        sr[1] = make_uint4(dep00, du * (unsigned)p.D, has_b ? (unsigned)(fw * p.D) : 0u, (unsigned)s.k);
        sr[2] = make_uint4((unsigned)my_a | ((unsigned)my_b << 16), __float_as_uint(s.wgt), __float_as_uint(s.dmean),
                           __float_as_uint(s.dsigma));
      }
      __syncwarp();
      if (q < total && lane == lo) sSmp[cl] += __popc(okm & seg);
    }
    if (q < total && lane == lo) {
      sLen[cl] = before + __popc(m1 & seg) + __popc(m2 & seg);
      sCnt[cl] += __popc(okm & seg);
    }
    __syncwarp();
  }
}

}  // namespace fbev
