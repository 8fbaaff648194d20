// tcgen05 GEMM fused with an all-gather of its A operand or a reduce-scatter of its
// output over NVLink peer memory (see teb200/comm.h for the protocol).  The GEMM
// pipeline is the one of gemm/gemm_tcgen05.cu (TMA producer warp, MMA warp, four
// epilogue warps, TMEM accumulators); this file adds
//   * copy CTAs that pull peer rows with L1-bypassing loads and publish per-block flags,
//   * a producer that waits (bounded) for the flag of the block it is about to load,
//   * an epilogue that stores tiles into the owner rank's staging buffer and a tail that
//     reduces the blocks this rank owns once every rank has delivered them.
// Tiles are visited in an order rotated by the rank so that at any time the ranks
// pull from / push to different peers.
#include <type_traits>

#include <teb200/comm.h>
#include <teb200/gemm_common.cuh>
#include <teb200/ptx.cuh>

namespace teb200 {
namespace {

using namespace gemm_detail;

constexpr int BN = 256;
// warp 0: TMA producer, warp 1: MMA issuer, warps 2..9: epilogue (two groups of four, one per 128-column half
// of the tile), warp 10: hands the staged half tiles to the copy engine and signals the owners
constexpr int kEpiWarps = 8;
constexpr int kEpiThreads = kEpiWarps * 32;
constexpr int kStoreWarp = 2 + kEpiWarps;
constexpr int kCommThreads = (kStoreWarp + 1) * 32;

struct CommParams {
  KernelParams k;
  int mode, rank, world;
  uint32_t* epoch_dev;   // calls completed on this (context, buffer slot); this call is number *epoch_dev + 1
  uint32_t* done_ctas;   // CTAs of this launch that have finished; the last one advances *epoch_dev
  int copy_ctas;
  int mb_per_rank;   // 128-row blocks owned by one rank
  int num_n;         // column tiles
  const uint8_t* a_full[kCommMaxRanks];
  const uint8_t* sfa_full[kCommMaxRanks];
  long long a_row_bytes, sf_bytes_per_mblock;
  uint32_t* ready[kCommMaxRanks];
  uint32_t* chunk_flags;
  uint8_t* stage[kCommMaxRanks];
  uint32_t* tile_flags[kCommMaxRanks];
  void* out;
  uint8_t* out_all[kCommMaxRanks];   // all-reduce: result buffers of every rank, else null
  uint32_t* ar_flags[kCommMaxRanks];
  int allreduce;
  SideGather side;
  int side_tma;  // the side gather's interleaved pieces leave through one 2-D TMA store each (rows <= 1 KB)
};

struct Tile {
  int mb, nb;
};

// Logical tile index -> (row block, column tile).  Row blocks are visited shard by shard,
// starting with the local shard (all-gather) or with the next rank's shard (reduce-scatter,
// own rows last); inside a shard the row block varies fastest.
__device__ __forceinline__ bool comm_tile(const CommParams& p, int t, Tile& out) {
  const int per_shard = p.mb_per_rank * p.num_n;
  if (t >= per_shard * p.world) return false;
  const int i = t / per_shard, r = t - i * per_shard;
  const int shard = p.mode == kCommAllGather ? (p.rank + i) % p.world : (p.rank + 1 + i) % p.world;
  out.mb = shard * p.mb_per_rank + r % p.mb_per_rank;
  out.nb = r / p.mb_per_rank;
  return true;
}

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long gtimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// Once any wait of this process has run out, the status word is set and the results are void anyway:
// later waits give up at once instead of each spending its full limit (a lost peer then costs about one
// limit per kernel, not one per tile).
__device__ __forceinline__ bool already_failed(const int* status) {
  return status != nullptr && *reinterpret_cast<const volatile int*>(status) != 0;
}
__device__ __forceinline__ bool wait_flag_ge_or_failed(const uint32_t* p, uint32_t want, const int* status) {
  if (ld_acquire_sys(p) >= want) return true;
  if (already_failed(status)) return false;
  return wait_flag_ge(p, want);
}

__device__ __forceinline__ bool wait_ge_gpu(const uint32_t* p, uint32_t want, const int* status = nullptr) {
  if (ld_acquire_gpu(p) >= want) return true;
  if (already_failed(status)) return false;
  const long long t0 = clock64();
  while (ld_acquire_gpu(p) < want) {
    if (clock64() - t0 > kWaitCycles) return false;
    __nanosleep(32);
  }
  return true;
}

// The call number lives in device memory so that a launch recorded in a CUDA graph stays correct on
// every replay: each CTA reads it on entry, and the CTA that finishes last stores the new value (all
// CTAs of the launch have read the old one by then; the next launch on the stream sees the new one).
__device__ __forceinline__ uint32_t read_epoch(const CommParams& p) {
  return *reinterpret_cast<const volatile uint32_t*>(p.epoch_dev) + 1u;
}
__device__ __forceinline__ void cta_done(const CommParams& p, uint32_t epoch) {
  __threadfence();
  if (atomicAdd(p.done_ctas, 1u) == gridDim.x - 1) {
    *reinterpret_cast<volatile uint32_t*>(p.done_ctas) = 0u;
    *reinterpret_cast<volatile uint32_t*>(p.done_ctas + 1) = 0u;  // the side gather's piece counter
    *reinterpret_cast<volatile uint32_t*>(p.epoch_dev) = epoch;
    __threadfence();
  }
}

// ---------------------------------------------------------------- copy CTAs (all-gather)
// One thread per copy CTA streams peer rows through a ring of shared-memory slots with bulk
// async copies: peer global -> shared (completion on an mbarrier), shared -> local global
// (bulk group).  About kCopySlots * kCopyPiece bytes stay in flight per CTA, which is what hides
// the NVLink round trip; plain per-thread loads keep only a few KB in flight.
constexpr int kCopyPiece = 32 * 1024;
constexpr int kCopySlots = 6;
constexpr int kHelperSlots = 4;  // ring of a GEMM CTA that joins the side gather: inside its pipeline stages

__device__ void copy_cta_loop(const CommParams& p, int cta, uint8_t* smem, uint64_t* bars, uint32_t epoch) {
  const int tid = threadIdx.x;
  if (cta == 0 && tid < p.world && tid != p.rank) {
    // this rank's rows were written by earlier kernels of this stream: publish them to every peer
    st_release_sys(p.ready[tid] + p.rank, epoch);
  }
  if (tid != 0 || p.mode != kCommAllGather) return;
  for (int i = 0; i < kCopySlots; ++i) mbar_init(&bars[i], 1);
  mbar_fence_init();
  const int items = (p.world - 1) * p.mb_per_rank;
  const long long data_bytes = static_cast<long long>(kBlockM) * p.a_row_bytes;
  const long long item_bytes = data_bytes + p.sf_bytes_per_mblock;
  const int pieces_per_item = static_cast<int>((data_bytes + kCopyPiece - 1) / kCopyPiece) +
                              static_cast<int>((p.sf_bytes_per_mblock + kCopyPiece - 1) / kCopyPiece);
  const int my_items = cta < items ? (items - cta + p.copy_ctas - 1) / p.copy_ctas : 0;
  const int total = my_items * pieces_per_item;
  (void)item_bytes;

  // piece index -> (source pointer, destination pointer, bytes, is last piece of its item, block id)
  auto piece = [&](int q, const uint8_t*& src, uint8_t*& dst, uint32_t& bytes, int& mb, int& srank) {
    const int it = cta + (q / pieces_per_item) * p.copy_ctas;
    const int j = q % pieces_per_item;
    srank = (p.rank + 1 + it / p.mb_per_rank) % p.world;
    mb = srank * p.mb_per_rank + it % p.mb_per_rank;
    const int data_pieces = static_cast<int>((data_bytes + kCopyPiece - 1) / kCopyPiece);
    if (j < data_pieces) {
      const long long off = static_cast<long long>(mb) * data_bytes + static_cast<long long>(j) * kCopyPiece;
      const long long left = data_bytes - static_cast<long long>(j) * kCopyPiece;
      bytes = static_cast<uint32_t>(left < kCopyPiece ? left : kCopyPiece);
      src = p.a_full[srank] + off;
      dst = const_cast<uint8_t*>(p.a_full[p.rank]) + off;
    } else {
      const int js = j - data_pieces;
      const long long off = static_cast<long long>(mb) * p.sf_bytes_per_mblock + static_cast<long long>(js) * kCopyPiece;
      const long long left = p.sf_bytes_per_mblock - static_cast<long long>(js) * kCopyPiece;
      bytes = static_cast<uint32_t>(left < kCopyPiece ? left : kCopyPiece);
      src = p.sfa_full[srank] + off;
      dst = const_cast<uint8_t*>(p.sfa_full[p.rank]) + off;
    }
  };

  bool ok = true;
  int issued = 0;
  auto issue_load = [&](int q) {
    const uint8_t* src; uint8_t* dst; uint32_t bytes; int mb, srank;
    piece(q, src, dst, bytes, mb, srank);
    if (q % pieces_per_item == 0) {
      // first piece of an item: the source rank must have published its rows for this call
      if (!wait_flag_ge_or_failed(p.ready[p.rank] + srank, epoch, p.k.status)) {
        if (p.k.status) atomicCAS(p.k.status, 0, kTimeoutPeerFlag);
      }
    }
    const int slot = q % kCopySlots;
    mbar_expect_tx(&bars[slot], bytes);
    bulk_load_1d(smem + slot * kCopyPiece, src, bytes, &bars[slot]);
  };
  for (; issued < total && issued < kCopySlots - 1; ++issued) issue_load(issued);
  for (int q = 0; q < total && ok; ++q) {
    const int slot = q % kCopySlots;
    const uint32_t phase = (q / kCopySlots) & 1;
    if (!mbar_wait(&bars[slot], phase)) {
      if (p.k.status) atomicCAS(p.k.status, 0, kTimeoutPeerFlag);
      ok = false;
    }
    const uint8_t* src; uint8_t* dst; uint32_t bytes; int mb, srank;
    piece(q, src, dst, bytes, mb, srank);
    if (ok) {
      bulk_store_1d(dst, smem + slot * kCopyPiece, bytes);
      tma_store_commit();
    }
    if (issued < total) {
      // the slot of piece `issued` was last read by the store of piece issued - kCopySlots = q - 1
      tma_store_wait_read<1>();
      issue_load(issued);
      ++issued;
    }
    if (q % pieces_per_item == pieces_per_item - 1) {
      // whole 128-row block landed: wait for the local writes, then publish the block
      tma_store_wait<0>();
      fence_proxy_async_all();
      __threadfence();
      st_release_gpu(p.chunk_flags + mb, epoch);
    }
  }
  if (!ok) {
    // never leave the GEMM waiting: publish every block of this CTA (data is wrong, status is set)
    tma_store_wait<0>();
    for (int it = cta; it < items; it += p.copy_ctas) {
      const int srank = (p.rank + 1 + it / p.mb_per_rank) % p.world;
      st_release_gpu(p.chunk_flags + srank * p.mb_per_rank + it % p.mb_per_rank, epoch);
    }
  }
}

// ---------------------------------------------------------------- side gather (bulk overlap)
// Run by warp 0 of every copy CTA after the gated gather.  A piece is up to 32 KB of whole rows of one
// rank's staged operand: one bulk load brings it into a shared-memory slot, then every lane stores the
// rows it owns to their (strided) place in the local gathered operand.  Scale chunks travel the same way
// as single-row pieces.
// Pieces are handed out by a device-wide counter, so that the GEMM CTAs can join once their tiles are done
// (their producer warp, over the freed pipeline stages): the gather then ends a few microseconds after the
// math instead of leaving 130 SMs idle while a dozen copy CTAs finish.  `bars` holds SLOTS mbarriers followed
// by SLOTS ints (the item that each slot carries).
template <int SLOTS>
__device__ void side_gather_loop(const CommParams& p, uint8_t* smem, uint64_t* bars, uint32_t epoch,
                                 const CUtensorMap* tmap_side) {
  const SideGather& g = p.side;
  if (g.rows <= 0) return;
  const int lane = threadIdx.x;  // caller guarantees threadIdx.x < 32
  int* slot_item = reinterpret_cast<int*>(bars + SLOTS);
  if (lane == 0) {
    for (int i = 0; i < SLOTS; ++i) mbar_init(&bars[i], 1);
    mbar_fence_init();
  }
  __syncwarp();
  const int rpp = kCopyPiece / g.row_bytes;                 // rows per piece
  const int data_pieces = (g.rows + rpp - 1) / rpp;
  const int sf_pieces = g.sf_chunk > 0 ? g.row_tiles : 0;
  const int per_rank = data_pieces + sf_pieces;
  const int items = p.world * per_rank;
  const long long data_bytes = static_cast<long long>(g.rows) * g.row_bytes;
  uint32_t* next_item = p.done_ctas + 1;  // reset by the CTA that finishes last (cta_done)

  // item -> source pointer, rows, bytes per row, destination of row 0, destination pitch
  auto piece = [&](int it, const uint8_t*& src, uint8_t*& dst, int& nrows, int& rbytes, long long& pitch, int& srank) {
    srank = (p.rank + 1 + it / per_rank) % p.world;  // own piece last
    const int j = it % per_rank;
    if (j < data_pieces) {
      const int r0 = j * rpp;
      nrows = g.rows - r0 < rpp ? g.rows - r0 : rpp;
      rbytes = g.row_bytes;
      src = g.src[srank] + static_cast<long long>(r0) * g.row_bytes;
      dst = g.dst + static_cast<long long>(srank) * g.dst_piece_off + static_cast<long long>(r0) * g.dst_pitch;
      pitch = g.dst_pitch;
    } else {
      const int t = j - data_pieces;
      nrows = 1;
      rbytes = g.sf_chunk;
      src = g.src[srank] + data_bytes + static_cast<long long>(t) * g.sf_chunk;
      dst = g.dst_sf + (static_cast<long long>(t) * p.world + srank) * g.sf_chunk;
      pitch = g.sf_chunk;
    }
  };
  int last_rank_ok = -1;
  // lane 0 only: claim the next item and start its load into the slot of piece number `n`; false: none left
  auto claim_and_load = [&](int n) -> bool {
    const int it = static_cast<int>(atomicAdd(next_item, 1u));
    if (it >= items) return false;
    const uint8_t* src; uint8_t* dst; int nrows, rbytes, srank; long long pitch;
    piece(it, src, dst, nrows, rbytes, pitch, srank);
    if (srank != p.rank && srank != last_rank_ok) {
      if (!wait_flag_ge_or_failed(p.ready[p.rank] + srank, epoch, p.k.status)) {
        if (p.k.status) atomicCAS(p.k.status, 0, kTimeoutPeerFlag);
      }
      last_rank_ok = srank;
    }
    const int slot = n % SLOTS;
    slot_item[slot] = it;
    const uint32_t bytes = static_cast<uint32_t>(nrows) * rbytes;
    mbar_expect_tx(&bars[slot], bytes);
    bulk_load_1d(smem + slot * kCopyPiece, src, bytes, &bars[slot]);
    return true;
  };
  int issued = 0;
  int more = 1;
  if (lane == 0) {
    while (issued < SLOTS - 1 && more) {
      if (claim_and_load(issued)) ++issued;
      else more = 0;
    }
  }
  __syncwarp();
  issued = __shfl_sync(0xffffffffu, issued, 0);
  more = __shfl_sync(0xffffffffu, more, 0);
  for (int q = 0; q < issued; ++q) {
    const int slot = q % SLOTS;
    const uint32_t phase = (q / SLOTS) & 1;
    if (!__all_sync(0xffffffffu, mbar_wait(&bars[slot], phase))) {
      if (lane == 0 && p.k.status) atomicCAS(p.k.status, 0, kTimeoutPeerFlag);
      break;
    }
    const int it = *reinterpret_cast<volatile int*>(&slot_item[slot]);
    const uint8_t* src; uint8_t* dst; int nrows, rbytes, srank; long long pitch;
    piece(it, src, dst, nrows, rbytes, pitch, srank);
    if (pitch == rbytes) {
      if (lane == 0) bulk_store_1d(dst, smem + slot * kCopyPiece, static_cast<uint32_t>(nrows) * rbytes);
    } else if (p.side_tma) {
      // the piece is a box of the gathered operand seen as [rows, pitch / 4] 32-bit words: one store request
      // instead of one per row (rows past the operand's end are clipped by the tensor map)
      if (lane == 0)
        tma_store_2d(tmap_side, smem + slot * kCopyPiece, static_cast<int>((dst - g.dst) % pitch) >> 2,
                     static_cast<int>((dst - g.dst) / pitch));
    } else {
      for (int r = lane; r < nrows; r += 32)
        bulk_store_1d(dst + static_cast<long long>(r) * pitch, smem + slot * kCopyPiece + r * rbytes, rbytes);
    }
    tma_store_commit();
    if (more) {
      // the slot of piece `issued` was last read by the stores of piece q - 1: every lane waits for its own
      tma_store_wait_read<1>();
      __syncwarp();
      int got = 0;
      if (lane == 0) got = claim_and_load(issued) ? 1 : 0;
      got = __shfl_sync(0xffffffffu, got, 0);
      if (got) ++issued;
      else more = 0;
    }
  }
  tma_store_wait<0>();
  __syncwarp();
}

// ---------------------------------------------------------------- reduce tail (reduce-scatter)
// Owner-side staging layout (written by the peers' bulk stores): one 64 KB record per
// (source rank, local row block, column tile); inside, two half tiles of 128 rows x 128
// columns, rows of 256 bytes whose 16-byte chunks are XOR-swizzled with (row & 7).
__device__ __forceinline__ size_t stage_tile_offset(const CommParams& p, int src, int mbl, int nb) {
  return ((static_cast<size_t>(src) * p.mb_per_rank + mbl) * p.num_n + nb) * 65536;
}

// Executed by the eight epilogue warps (kEpiThreads threads, named barrier 1) after their tile loop.  A thread
// keeps U vectors x world sources (about eight 16-byte loads) in flight, which is what lets the tail run near
// the memory rate instead of at one DRAM round trip per vector.
template <typename T, int U, int WMAX>
__device__ void reduce_tail(const CommParams& p, int cta, int num_ctas, int et, uint32_t epoch) {
  const int items = p.mb_per_rank * p.num_n;
  const uint32_t expected = epoch * static_cast<uint32_t>(p.num_n) * 2u;  // two half tiles per tile
  const uint8_t* stage = p.stage[p.rank];
  T* out = reinterpret_cast<T*>(p.out);
  const int N = p.k.N;
  constexpr bool kBf = sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value;
  for (int it = cta; it < items; it += num_ctas) {
    const int mbl = it % p.mb_per_rank, nb = it / p.mb_per_rank;
    if (et < p.world) {
      // one waiter per source rank
      if (!wait_flag_ge_or_failed(p.tile_flags[p.rank] + et * p.mb_per_rank + mbl, expected, p.k.status)) {
        if (p.k.status) atomicCAS(p.k.status, 0, kTimeoutPeerFlag);
      }
    }
    named_bar_sync(1, kEpiThreads);
    const int c_lo = nb * BN;
    const uint8_t* tile0 = stage + stage_tile_offset(p, 0, mbl, nb);
    const size_t src_pitch = stage_tile_offset(p, 1, 0, 0);
    for (int v0 = et; v0 < kBlockM * 32; v0 += kEpiThreads * U) {
      uint4 raw[U][WMAX];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int v = v0 + u * kEpiThreads;
        const int r = v >> 5, cv = v & 31;  // row, 8-column vector index inside the 256-column tile
        const int half = cv >> 4, chunk = (cv & 15) ^ (r & 7);
        const size_t in_tile = static_cast<size_t>(half) * 32768 + static_cast<size_t>(r) * 256 + chunk * 16;
#pragma unroll
        for (int sr = 0; sr < WMAX; ++sr)
          if (sr < p.world) raw[u][sr] = __ldcg(reinterpret_cast<const uint4*>(tile0 + sr * src_pitch + in_tile));
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int v = v0 + u * kEpiThreads;
        const int r = v >> 5, cv = v & 31;
        const int c = c_lo + cv * 8;
        if (c >= N) continue;
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0.f;
#pragma unroll
        for (int sr = 0; sr < WMAX; ++sr) {
          if (sr < p.world) {
            const uint32_t w[4] = {raw[u][sr].x, raw[u][sr].y, raw[u][sr].z, raw[u][sr].w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (kBf) {
                acc[2 * j] += __uint_as_float(w[j] << 16);
                acc[2 * j + 1] += __uint_as_float(w[j] & 0xFFFF0000u);
              } else {
                const __half2 h = *reinterpret_cast<const __half2*>(&w[j]);
                acc[2 * j] += __low2float(h);
                acc[2 * j + 1] += __high2float(h);
              }
            }
          }
        }
        if (p.k.bias != nullptr) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float b;
            if (p.k.bias_dtype == kFloat32) b = reinterpret_cast<const float*>(p.k.bias)[c + i];
            else if (p.k.bias_dtype == kBFloat16) b = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.k.bias)[c + i]);
            else b = __half2float(reinterpret_cast<const __half*>(p.k.bias)[c + i]);
            acc[i] += b;
          }
        }
        uint4 o;
        if (kBf) {
          o = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]),
                         pack_bf16x2(acc[6], acc[7]));
        } else {
          o = make_uint4(pack_f16x2(acc[0], acc[1]), pack_f16x2(acc[2], acc[3]), pack_f16x2(acc[4], acc[5]),
                         pack_f16x2(acc[6], acc[7]));
        }
        if (!p.allreduce) {
          *reinterpret_cast<uint4*>(out + static_cast<size_t>(mbl * kBlockM + r) * N + c) = o;
        } else {
          // the reduced row goes to its place in the full result of every rank
          const size_t at = (static_cast<size_t>(p.rank) * p.mb_per_rank * kBlockM + mbl * kBlockM + r) * N + c;
#pragma unroll
          for (int dr = 0; dr < WMAX; ++dr)
            if (dr < p.world) *reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.out_all[dr]) + at) = o;
        }
      }
    }
    named_bar_sync(1, kEpiThreads);
  }
  if (p.allreduce) {
    // this CTA's rows are on their way: tell every rank, then wait until every rank's CTAs have told us
    __threadfence_system();
    named_bar_sync(1, kEpiThreads);
    if (et < p.world) red_release_sys_add(p.ar_flags[et] + p.rank, 1u);
    if (et < p.world) {
      if (!wait_flag_ge_or_failed(p.ar_flags[p.rank] + et, epoch * static_cast<uint32_t>(num_ctas), p.k.status)) {
        if (p.k.status) atomicCAS(p.k.status, 0, kTimeoutPeerFlag);
      }
    }
    named_bar_sync(1, kEpiThreads);
  }
}

template <typename T>
__device__ __forceinline__ void reduce_tail_any(const CommParams& p, int cta, int num_ctas, int et, uint32_t epoch) {
  if (p.world <= 2) reduce_tail<T, 4, 2>(p, cta, num_ctas, et, epoch);
  else if (p.world <= 4) reduce_tail<T, 2, 4>(p, cta, num_ctas, et, epoch);
  else reduce_tail<T, 1, kCommMaxRanks>(p, cta, num_ctas, et, epoch);
}

// Shared-memory plan: one pipeline stage is traded for a 64 KB output staging area (two half tiles) from
// which the epilogue's stores leave: 32 KB bulk stores to the owner rank (reduce-scatter) or TMA stores of
// 128-byte-swizzled boxes to the local output (all-gather).
template <int KIND, int MODE>
struct CommSmem {
  using C = Cfg<KIND, BN>;
  static constexpr int kStagingBytes = 2 * 32768;
  static constexpr int kStages = 3;
  static constexpr int kBytes = kStages * C::kStageBytes + kStagingBytes + 1024 + 1024;
  static_assert(kBytes <= 227 * 1024, "shared memory plan exceeds the per-CTA limit");
  static_assert(kHelperSlots * kCopyPiece <= kStages * C::kStageBytes, "helper ring must fit in the pipeline stages");
  static_assert(kCopySlots * kCopyPiece <= kStages * C::kStageBytes + kStagingBytes,
                "copy ring must fit in front of the barriers");
};

template <int KIND, int MODE>
__global__ void __launch_bounds__(kCommThreads, 1)
comm_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_d, const __grid_constant__ CUtensorMap tmap_side,
                 const CommParams p) {
  using C = Cfg<KIND, BN>;
  constexpr int NS = CommSmem<KIND, MODE>::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = smem + NS * C::kStageBytes;  // two 32 KB half-tile buffers of the epilogue
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + CommSmem<KIND, MODE>::kStagingBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + NS;
  uint64_t* tfull_bar = bars + 2 * NS;
  uint64_t* tempty_bar = tfull_bar + C::kAccStages;
  uint64_t* staged_bar = tempty_bar + C::kAccStages;  // [2] epilogue group -> store warp: half tile is in shared memory
  uint64_t* free_bar = staged_bar + 2;                // [2] store warp -> epilogue group: staging buffer may be rewritten
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(free_bar + 2);
  unsigned long long* dbg = reinterpret_cast<unsigned long long*>(p.k.aux);  // optional [grid, 4] timestamps

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  int gemm_ctas = gridDim.x, gemm_cta = blockIdx.x;
  if (p.copy_ctas > 0) {
    gemm_ctas = gridDim.x - p.copy_ctas;
    gemm_cta = blockIdx.x - p.copy_ctas;
    if (static_cast<int>(blockIdx.x) < p.copy_ctas) {
      const uint32_t ep = read_epoch(p);
      if (warp == 0) {
        if (dbg && lane == 0) dbg[blockIdx.x * 4 + 0] = gtimer();
        copy_cta_loop(p, blockIdx.x, smem, bars, ep);  // publishes this rank's rows; gated gather (all-gather mode)
        __syncwarp();
        if (dbg && lane == 0) dbg[blockIdx.x * 4 + 1] = gtimer();
        side_gather_loop<kCopySlots>(p, smem, bars + kCopySlots, ep, &tmap_side);
        if (dbg && lane == 0) dbg[blockIdx.x * 4 + 2] = gtimer();
        if (lane == 0) cta_done(p, ep);
      }
      return;  // copy CTAs never touch TMEM or the pipeline barriers
    }
  }
  const int num_k_blocks = (p.k.K + C::kBlockK - 1) / C::kBlockK;
  const uint32_t epoch = read_epoch(p);

  if (threadIdx.x == 0) {
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
    for (int i = 0; i < NS; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < C::kAccStages; ++i) {
      mbar_init(&tfull_bar[i], 1);
      mbar_init(&tempty_bar[i], kEpiWarps);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&staged_bar[i], 4);
      mbar_init(&free_bar[i], 1);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_sfa = tmem_base + C::kAccStages * BN;
  const uint32_t tmem_sfb = tmem_sfa + C::kSfaCols;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    bool helper_ok = false;
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      Tile ti;
      for (int t = gemm_cta; ok && comm_tile(p, t, ti); t += gemm_ctas) {
        if (MODE == kCommAllGather && ti.mb / p.mb_per_rank != p.rank) {
          // rows of a peer: wait until a copy CTA has landed this 128-row block in local memory
          if (!wait_ge_gpu(p.chunk_flags + ti.mb, epoch, p.k.status)) {
            if (p.k.status) atomicCAS(p.k.status, 0, kTimeoutPeerFlag);
          }
          fence_proxy_async_all();  // generic-proxy writes of the copy CTA -> TMA (async proxy) reads
        }
        const int m0 = ti.mb * kBlockM, n0 = ti.nb * BN;
        for (int kb = 0; kb < num_k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
            if (p.k.status) atomicCAS(p.k.status, 0, kTimeoutProducer);
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * C::kStageBytes;
          uint8_t* sb = sa + C::kABytes;
          mbar_expect_tx(&full_bar[stage], C::kABytes + C::kBBytes + C::kSfaBytes + C::kSfbBytes);
          if constexpr (KIND == kKindF16) {
            tma_load_2d(sa, &tmap_a, &full_bar[stage], kb * C::kBlockK, m0);
            tma_load_2d(sb, &tmap_b, &full_bar[stage], kb * C::kBlockK, n0);
          } else {
            const int kbyte0 = kb * C::kBlockKBytes;
            tma_load_2d(sa, &tmap_a, &full_bar[stage], kbyte0, m0);
            tma_load_2d(sb, &tmap_b, &full_bar[stage], kbyte0, n0);
            uint8_t* ssfa = sb + C::kBBytes;
            uint8_t* ssfb = ssfa + C::kSfaBytes;
            bulk_load_1d(ssfa, p.k.sfa + (static_cast<size_t>(ti.mb) * p.k.sf_k_tiles + kb) * 512, 512,
                         &full_bar[stage]);
#pragma unroll
            for (int j = 0; j < BN / 128; ++j)
              bulk_load_1d(ssfb + j * 512,
                           p.k.sfb + (static_cast<size_t>(n0 / 128 + j) * p.k.sf_k_tiles + kb) * 512, 512,
                           &full_bar[stage]);
          }
          if (++stage == NS) { stage = 0; phase ^= 1; }
        }
      }
      if (p.side.rows > 0) {
        // every stage has been consumed by the tensor core: the pipeline's shared memory is free
        for (int i = 0; ok && i < NS; ++i) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
            if (p.k.status) atomicCAS(p.k.status, 0, kTimeoutProducer);
            ok = false;
          }
          if (++stage == NS) { stage = 0; phase ^= 1; }
        }
        helper_ok = ok;
      }
    }
    if (p.side.rows > 0) {
      // join the side gather with the pieces that the copy CTAs have not claimed yet
      helper_ok = __shfl_sync(0xffffffffu, helper_ok ? 1 : 0, 0) != 0;
      if (helper_ok) side_gather_loop<kHelperSlots>(p, smem, bars + 32, epoch, &tmap_side);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // The whole warp walks the loop (values stay warp-uniform); one elected lane issues.
    {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      Tile ti;
      for (int t = gemm_cta; ok && comm_tile(p, t, ti); t += gemm_ctas) {
        if (!__all_sync(0xffffffffu, mbar_wait(&tempty_bar[acc], acc_phase ^ 1))) {
          if (lane == 0 && p.k.status) atomicCAS(p.k.status, 0, kTimeoutMma);
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = 0; kb < num_k_blocks; ++kb) {
          if (!__all_sync(0xffffffffu, mbar_wait(&full_bar[stage], phase))) {
            if (lane == 0 && p.k.status) atomicCAS(p.k.status, 0, kTimeoutMma);
            ok = false;
            break;
          }
          tc_fence_after();
          if (elect_one()) {
          const uint32_t sa = smem_u32(smem + stage * C::kStageBytes);
          const uint32_t sb = sa + C::kABytes;
          const uint64_t adesc = umma_desc_k_sw128(sa);
          const uint64_t bdesc = umma_desc_k_sw128(sb);
          if constexpr (KIND == kKindF16) {
#pragma unroll
            for (int k = 0; k < 4; ++k) umma_f16(tmem_d, adesc + k * 2, bdesc + k * 2, p.k.idesc, (kb | k) != 0);
          } else {
            const uint32_t ssfa = sb + C::kBBytes;
            const uint32_t ssfb = ssfa + C::kSfaBytes;
            utccp_sf(tmem_sfa, umma_desc_sf(ssfa));
#pragma unroll
            for (int j = 0; j < BN / 128; ++j) utccp_sf(tmem_sfb + j * 4, umma_desc_sf(ssfb + j * 512));
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const uint32_t idesc = p.k.idesc | (uint32_t(k) << 29) | (uint32_t(k) << 4);
              umma_mxf8(tmem_d, adesc + k * 2, bdesc + k * 2, idesc, (kb | k) != 0, tmem_sfa, tmem_sfb);
            }
          }
          tc_commit(&empty_bar[stage]);
          }
          __syncwarp();
          if (++stage == NS) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        if (elect_one()) tc_commit(&tfull_bar[acc]);
        __syncwarp();
        if (++acc == C::kAccStages) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else if (warp < kStoreWarp) {
    // ------------------------------------------------------------ epilogue (warps 2..9)
    // Group g (four warps) owns columns [128 g, 128 g + 128) of every tile.  A thread pulls its 128 accumulator
    // values with four back-to-back TMEM loads and ONE wait, and the accumulator is released right away (all
    // eight warps have read it by then): the tensor core waits for a TMEM read, never for a store.  The values
    // are then packed into the group's 32 KB staging buffer and handed to the store warp through an mbarrier.
    const int quarter = warp & 3;              // TMEM lanes this warp may read
    const int g = (warp - 2) >> 2;             // column half
    const int row = quarter * 32 + lane;       // row inside the tile
    const int et = (warp - 2) * 32 + lane;     // 0..255 inside the epilogue group
    int acc = 0;
    uint32_t acc_phase = 0;
    const float alpha = p.k.alpha * (p.k.alpha_dev ? *p.k.alpha_dev : 1.0f);
    const bool bf = p.k.d_dtype == kBFloat16;
    if (dbg && et == 0) dbg[blockIdx.x * 4 + 0] = gtimer();
    const int sw = row & 7;
    uint8_t* buf = staging + g * 32768;
    uint32_t n_local = 0;  // tiles handled so far
    bool dead = false;     // a wait ran out: keep walking and arriving (others wait on us), wait no more
    Tile ti;
    for (int t = gemm_cta; comm_tile(p, t, ti); t += gemm_ctas, ++n_local) {
      if (!dead && !mbar_wait(&tfull_bar[acc], acc_phase)) {
        if (lane == 0 && p.k.status) atomicCAS(p.k.status, 0, kTimeoutEpilogue);
        dead = true;
      }
      tc_fence_after();
      const int n0 = ti.nb * BN;
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + acc * BN + g * 128;
      uint32_t r[4][32];
#pragma unroll
      for (int j = 0; j < 4; ++j) tmem_ld_32x32(taddr + j * 32, r[j]);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      // the store of the previous tile has read this group's staging buffer
      if (!dead && !mbar_wait(&free_bar[g], (n_local & 1) ^ 1)) {
        if (lane == 0 && p.k.status) atomicCAS(p.k.status, 0, kTimeoutEpilogue);
        dead = true;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[j][i]) * alpha;
        if (MODE == kCommAllGather && p.k.bias != nullptr) {
          const int col0 = n0 + g * 128 + j * 32;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (col0 + i < p.k.N) {
              float b;
              if (p.k.bias_dtype == kFloat32) b = reinterpret_cast<const float*>(p.k.bias)[col0 + i];
              else if (p.k.bias_dtype == kBFloat16)
                b = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.k.bias)[col0 + i]);
              else b = __half2float(reinterpret_cast<const __half*>(p.k.bias)[col0 + i]);
              v[i] += b;
            }
          }
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int i = 8 * c;
          uint4 o;
          if (bf) {
            o = make_uint4(pack_bf16x2(v[i], v[i + 1]), pack_bf16x2(v[i + 2], v[i + 3]), pack_bf16x2(v[i + 4], v[i + 5]),
                           pack_bf16x2(v[i + 6], v[i + 7]));
          } else {
            o = make_uint4(pack_f16x2(v[i], v[i + 1]), pack_f16x2(v[i + 2], v[i + 3]), pack_f16x2(v[i + 4], v[i + 5]),
                           pack_f16x2(v[i + 6], v[i + 7]));
          }
          const int chunk = j * 4 + c;  // 16-byte chunk of this thread's 256 bytes (128 columns)
          if (MODE == kCommReduceScatter) {
            // owner-side layout: rows of 256 bytes, chunks XOR-swizzled with (row & 7)
            *reinterpret_cast<uint4*>(buf + row * 256 + ((chunk ^ sw) << 4)) = o;
          } else {
            // two TMA boxes of 128 rows x 128 bytes (64 columns each), 128-byte swizzle
            *reinterpret_cast<uint4*>(buf + (chunk >> 3) * 16384 + row * 128 + (((chunk & 7) ^ sw) << 4)) = o;
          }
        }
      }
      fence_proxy_async_smem();  // generic-proxy writes to shared memory -> bulk / TMA (async proxy) read
      __syncwarp();
      if (lane == 0) mbar_arrive(&staged_bar[g]);
      if (++acc == C::kAccStages) { acc = 0; acc_phase ^= 1; }
    }
    if (dbg && et == 0) dbg[blockIdx.x * 4 + 1] = gtimer();
    if (MODE == kCommReduceScatter) {
      if (p.k.d_dtype == kBFloat16) reduce_tail_any<__nv_bfloat16>(p, gemm_cta, gemm_ctas, et, epoch);
      else reduce_tail_any<__half>(p, gemm_cta, gemm_ctas, et, epoch);
      if (dbg && et == 0) dbg[blockIdx.x * 4 + 3] = gtimer();
    }
  } else if (lane == 0) {
    // ------------------------------------------------------------ store warp (one thread)
    // Hands every staged half tile to the copy engine: a 32 KB bulk store into the owner rank's staging
    // buffer (reduce-scatter) or two TMA box stores to the local output (all-gather).  A staging buffer is
    // given back as soon as its store has READ it.  The owner's counter is bumped one tile later, when the
    // stores it announces have completed, so that neither NVLink latency nor the release fence sits between
    // two tiles of the epilogue warps.
    uint32_t n_local = 0;
    uint32_t* prev_flag = nullptr;
    bool dead = false;
    Tile ti;
    for (int t = gemm_cta; comm_tile(p, t, ti); t += gemm_ctas, ++n_local) {
      const int m0 = ti.mb * kBlockM, n0 = ti.nb * BN;
      uint8_t* dst_tile = nullptr;
      uint32_t* flag = nullptr;
      if (MODE == kCommReduceScatter) {
        const int owner = ti.mb / p.mb_per_rank, mbl = ti.mb % p.mb_per_rank;
        dst_tile = p.stage[owner] + stage_tile_offset(p, p.rank, mbl, ti.nb);
        flag = p.tile_flags[owner] + p.rank * p.mb_per_rank + mbl;
      }
#pragma unroll 1
      for (int g = 0; g < 2; ++g) {
        if (!dead && !mbar_wait(&staged_bar[g], n_local & 1)) {
          if (p.k.status) atomicCAS(p.k.status, 0, kTimeoutEpilogue);
          dead = true;
        }
        const uint8_t* buf = staging + g * 32768;
        if (MODE == kCommReduceScatter) {
          bulk_store_1d(dst_tile + g * 32768, buf, 32768);
        } else {
#pragma unroll
          for (int b = 0; b < 2; ++b) {
            const int col = n0 + g * 128 + b * 64;
            if (col < p.k.N) tma_store_2d(&tmap_d, buf + b * 16384, col, m0);  // clipped at the matrix edge
          }
        }
        tma_store_commit();
      }
      tma_store_wait_read<1>();
      mbar_arrive(&free_bar[0]);
      tma_store_wait_read<0>();
      mbar_arrive(&free_bar[1]);
      if (MODE == kCommReduceScatter) {
        if (prev_flag != nullptr) {
          tma_store_wait<2>();       // everything but this tile's two stores has completed
          fence_proxy_async_all();   // async-proxy writes (the bulk stores) before the generic-proxy release
          red_release_sys_add(prev_flag, 2u);
        }
        prev_flag = flag;
      }
    }
    tma_store_wait<0>();  // every store has completed (shared memory may go, data is at its place)
    if (dbg) dbg[blockIdx.x * 4 + 2] = gtimer();
    if (MODE == kCommReduceScatter && prev_flag != nullptr) {
      fence_proxy_async_all();
      red_release_sys_add(prev_flag, 2u);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
  if (threadIdx.x == 0) cta_done(p, epoch);
}

template <int KIND, int MODE>
cudaError_t launch_comm(const CommGemmArgs& a, cudaStream_t stream) {
  using C = Cfg<KIND, BN>;
  const GemmArgs& g = a.g;
  CUtensorMap ta, tb;
  bool ok;
  if (KIND == kKindF16) {
    ok = make_tensor_map_2d(&ta, g.a, g.a_dtype, g.M, g.K, g.lda, kBlockM, 64, true) &&
         make_tensor_map_2d(&tb, g.b, g.b_dtype, g.N, g.K, g.ldb, BN, 64, true);
  } else {
    ok = make_tensor_map_2d(&ta, g.a, kByte, g.M, g.K, g.lda, kBlockM, 128, true) &&
         make_tensor_map_2d(&tb, g.b, kByte, g.N, g.K, g.ldb, BN, 128, true);
  }
  // all-gather mode stores the output through TMA boxes of 128 rows x 64 16-bit columns
  CUtensorMap td = ta;
  if (MODE == kCommAllGather)
    ok = ok && make_tensor_map_2d(&td, g.d, g.d_dtype, g.M, g.N, g.ldd, 128, 64, true);
  if (!ok) return cudaErrorInvalidValue;
  CommParams p = {};
  KernelParams& k = p.k;
  k.d = g.d; k.bias = g.bias; k.aux = g.aux; k.sfa = g.sfa; k.sfb = g.sfb; k.alpha_dev = g.alpha_dev;
  k.group_offsets = nullptr; k.status = g.status; k.alpha = g.alpha;
  k.M = g.M; k.N = g.N; k.K = g.K; k.ldd = g.ldd;
  k.d_dtype = g.d_dtype; k.bias_dtype = g.bias_dtype; k.epilogue = 0; k.accumulate = 0; k.a_mn = 0; k.b_mn = 0;
  k.idesc = make_idesc(KIND, g.a_dtype, g.b_dtype, BN, false, false);
  k.num_groups = 0;
  k.sf_k_tiles = KIND == kKindF16 ? 0 : ((g.K + 31) / 32 + 3) / 4;
  p.mode = MODE; p.rank = a.rank; p.world = a.world; p.epoch_dev = a.epoch_dev; p.done_ctas = a.epoch_dev + 1;
  p.mb_per_rank = g.M / kBlockM / a.world;
  p.num_n = (g.N + BN - 1) / BN;
  const int sms = g.sm_count > 0 ? g.sm_count : device_sm_count();
  const bool side = a.side.rows > 0;
  int copy = (MODE == kCommAllGather || side) ? a.copy_ctas : 0;
  if (copy < 1 && (MODE == kCommAllGather || side)) copy = 1;
  if (copy > sms / 2) copy = sms / 2;
  p.copy_ctas = copy;
  p.side = a.side;
  CUtensorMap ts = ta;
  if (side) {
    if (a.side.row_bytes <= 0 || a.side.row_bytes % 16 != 0 || a.side.row_bytes > kCopyPiece ||
        a.side.sf_chunk % 16 != 0 || a.side.sf_chunk > kCopyPiece || a.side.dst == nullptr ||
        a.side.dst_pitch % 16 != 0 || a.side.dst_piece_off % 16 != 0 ||
        reinterpret_cast<uintptr_t>(a.side.dst) % 16 != 0 || (a.side.sf_chunk > 0 && a.side.dst_sf == nullptr))
      return cudaErrorInvalidValue;
    for (int r = 0; r < a.world; ++r)
      if (a.side.src[r] == nullptr || a.ready[r] == nullptr || reinterpret_cast<uintptr_t>(a.side.src[r]) % 16 != 0)
        return cudaErrorInvalidValue;
    if (a.side.dst_pitch != a.side.row_bytes && a.side.row_bytes <= 1024 && a.side.dst_pitch % a.side.row_bytes == 0) {
      const int rpp = kCopyPiece / a.side.row_bytes;  // rows per piece (32..256)
      p.side_tma = rpp <= 256 &&
                   make_tensor_map_2d(&ts, a.side.dst, kFloat32, a.side.rows, a.side.dst_pitch / 4, a.side.dst_pitch / 4,
                                      rpp, a.side.row_bytes / 4, false);
    }
  }
  for (int r = 0; r < kCommMaxRanks; ++r) {
    p.a_full[r] = a.a_full[r]; p.sfa_full[r] = a.sfa_full[r]; p.ready[r] = a.ready[r];
    p.stage[r] = a.stage[r]; p.tile_flags[r] = a.tile_flags[r];
  }
  p.a_row_bytes = a.a_row_bytes; p.sf_bytes_per_mblock = a.sf_bytes_per_mblock;
  p.chunk_flags = a.chunk_flags; p.out = a.out;
  p.allreduce = a.mode == kCommAllReduce ? 1 : 0;
  for (int r = 0; r < kCommMaxRanks; ++r) {
    p.out_all[r] = a.out_all[r];
    p.ar_flags[r] = a.ar_flags[r];
  }
  if (p.allreduce)
    for (int r = 0; r < a.world; ++r)
      if (a.out_all[r] == nullptr || a.ar_flags[r] == nullptr) return cudaErrorInvalidValue;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(comm_gemm_kernel<KIND, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         CommSmem<KIND, MODE>::kBytes);
    if (e != cudaSuccess) return e;
    // the protocol needs every CTA of the grid resident at once: refuse a configuration that cannot be
    int per_sm = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, comm_gemm_kernel<KIND, MODE>, kCommThreads,
                                                      CommSmem<KIND, MODE>::kBytes);
    if (e != cudaSuccess) return e;
    if (per_sm < 1) return cudaErrorLaunchOutOfResources;
    attr_set = true;
  }
  // every CTA must be resident at once (copy CTAs and GEMM CTAs wait on one another; the
  // reduce tail waits on peers): one CTA per SM, never more CTAs than SMs
  comm_gemm_kernel<KIND, MODE><<<sms, kCommThreads, CommSmem<KIND, MODE>::kBytes, stream>>>(ta, tb, td, ts, p);
  return cudaGetLastError();
}

}  // namespace

cudaError_t comm_gemm(const CommGemmArgs& a, cudaStream_t stream) {
  const GemmArgs& g = a.g;
  if (a.world < 2 || a.world > kCommMaxRanks || a.epoch_dev == nullptr) return cudaErrorInvalidValue;
  if (g.M % (kBlockM * a.world) != 0 || g.N % 8 != 0 || g.K <= 0) return cudaErrorInvalidValue;
  if (g.d_dtype != kBFloat16 && g.d_dtype != kFloat16) return cudaErrorInvalidValue;
  const bool mx = g.sfa != nullptr;
  if (mx && g.K % 128 != 0) return cudaErrorInvalidValue;
  if (a.mode == kCommAllGather)
    return mx ? launch_comm<kKindMxf8, kCommAllGather>(a, stream) : launch_comm<kKindF16, kCommAllGather>(a, stream);
  if (a.mode == kCommReduceScatter || a.mode == kCommAllReduce)
    return mx ? launch_comm<kKindMxf8, kCommReduceScatter>(a, stream)
              : launch_comm<kKindF16, kCommReduceScatter>(a, stream);
  return cudaErrorInvalidValue;
}

}  // namespace teb200
