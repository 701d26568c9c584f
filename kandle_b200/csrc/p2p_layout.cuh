// Layout of the per-rank exchange buffer that peers map through CUDA IPC, shared by the one-shot
// all-reduce (p2p_allreduce.cu) and the tensor-parallel form of the fused decode layer kernel
// (decode_layer.cu).
//
//   [0, 2 MiB)          data slot 0      all-reduce: calls with an even counter
//   [2 MiB, 4 MiB)      data slot 1      all-reduce: calls with an odd counter
//   [4 MiB, 6 MiB)      data slot 2      layer kernel: partial sums of o_proj
//   [6 MiB, 8 MiB)      data slot 3      layer kernel: partial sums of down_proj
//   then                flags of the all-reduce        [2 slots][128 rows][8 ranks]  uint32 tags
//   then                flags of the layer kernel      [2 phases][128 units][8 ranks] uint32 tags
// Each kernel has its own slots, flags and tag counter, so calls of the two may be mixed on a stream.
//
// Why two slots are enough for the layer kernel: a rank rewrites its o_proj slot in its NEXT launch;
// it left the previous launch only after every peer had published all its down_proj flags, and a
// peer publishes those only after all its units finished the o_proj phase (reads included).  It
// rewrites its down_proj slot only after its next o_proj phase completed, which needs every peer's
// o_proj flags of that next launch: the peer's previous launch has ended by then.
#pragma once
#include <cstddef>
#include <cstdint>

namespace kd {

constexpr int P2P_MAX_RANKS = 8;
constexpr int P2P_MAX_ROWS = 128;
constexpr size_t P2P_SLOT_BYTES = 2u << 20;
constexpr size_t P2P_LAYER_SLOT_OFFSET = 2 * P2P_SLOT_BYTES;
constexpr size_t P2P_FLAG_OFFSET = 4 * P2P_SLOT_BYTES;
constexpr size_t P2P_FLAG_BYTES = 2 * P2P_MAX_ROWS * P2P_MAX_RANKS * sizeof(unsigned);
constexpr size_t P2P_LAYER_FLAG_OFFSET = P2P_FLAG_OFFSET + P2P_FLAG_BYTES;
constexpr size_t P2P_BUF_BYTES = P2P_LAYER_FLAG_OFFSET + P2P_FLAG_BYTES;
constexpr long long P2P_WAIT_CYCLES = 10000000000LL;        // about five seconds: ranks are separate processes

// State a kernel needs to talk to its peers (filled by p2p_allreduce.cu).
struct P2pPeers {
  char* buf[P2P_MAX_RANKS];
  int nranks, rank;
  unsigned* layer_seq;      // device call counter of the layer kernel (+1: its completion ticket)
  long long wait_cycles;    // bound of every wait on a peer's flag
};
// KD_OK and *out filled when peer buffers are connected across processes, or to silent stand-ins
// (kd_p2p_selftest_silent_peers); not in emulation mode.
int p2p_peers(P2pPeers* out);

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_peer_f4(const float4* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}

}  // namespace kd
