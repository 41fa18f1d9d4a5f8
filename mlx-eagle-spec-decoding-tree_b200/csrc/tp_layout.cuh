// Layout of a tensor-parallel exchange buffer (one per GPU, mapped by every process of the group).
// Header: flag lines and counters of the two users, then the key slots of the argmax combine; after the
// header two buffers of [32][hidden] fp32 partial products, used in turn, then two gather areas of [32][hidden] fp16
// (the reduced hidden states of the two-shot exchange), used in turn, then two sets, used in turn, of kMaxTp slots
// of [32][hidden] fp32: slot r of a set holds the partial products rank r stored here (push form of the exchange).
#pragma once

namespace b200 {

constexpr int kMaxTp = 8;             // GPUs of one tensor-parallel group
constexpr int kTpFlagStride = 64;     // one line per peer: peer r raises the word at r * 64
constexpr int kTpFwdArrive = 0;       // persistent forward kernel: arrivals of all CTAs of all GPUs (remote atomics)
constexpr int kTpFwdCount = 512;      //   exchanges completed by earlier launches (local word)
constexpr int kTpFwdLocal = 768;      //   tickets of this GPU's own CTAs for the all-GPU barrier (local atomics)
constexpr int kTpKeyFlags = 1024;     // argmax combine: flags written by the peers
constexpr int kTpKeyCount = 1536;     //   combines completed so far (local word)
constexpr int kTpKeyErr = 1540;       //   non-zero after a combine whose wait for a peer gave up
constexpr int kTpKeys = 2048;         //   [2][32] 64-bit keys, the two halves used in turn
constexpr int kTpHeader = 4096;       // partial products start here

struct TpPeers {
    unsigned char* p[kMaxTp];         // p[r] = rank r's exchange buffer as mapped into this process
};

__device__ __forceinline__ void st_release_sys(unsigned* q, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(q), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* q) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(q) : "memory");
    return v;
}

}  // namespace b200
