// Copies from global to shared memory that do not pass through registers (cp.async).  Copies issued by a thread
// are closed into a group with copies_commit(); copies_wait<N>() returns when at most N of the thread's groups
// are still in flight (groups complete in order).  What another thread copied is visible after a barrier that
// follows that thread's wait.
#pragma once

namespace dlgo {

// 16 bytes; both addresses 16-byte aligned
__device__ __forceinline__ void copy16_async(float* dst_shared, const float* src) {
  const unsigned dst = (unsigned)__cvta_generic_to_shared(dst_shared);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
// 4 bytes, for rows whose pieces do not start on 16-byte boundaries
__device__ __forceinline__ void copy4_async(float* dst_shared, const float* src) {
  const unsigned dst = (unsigned)__cvta_generic_to_shared(dst_shared);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void copies_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void copies_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

}  // namespace dlgo
