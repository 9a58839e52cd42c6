// Output exchange of a head-sharded prompt by the GPU's copy engines.
//
// When the KV heads of a layer are split over the GPUs of one node, every GPU ends a layer holding the
// output rows of its own heads inside its [B, L, H, D] buffer; the other GPUs need them too.  The
// prefill kernels can store the rows into the peers themselves (kb200_out_fanout), but from four GPUs
// on the NVLink time of a reuse layer exceeds its compute time and the stores hold the kernel up.  The
// calls here take the exchange off the kernels' critical path: the kernel writes only its own buffer,
// and the slice is then copied into every peer's buffer by the DMA engines (one copy per peer, each on a
// stream of its own: a strided 2-D copy for [B, L, H, D] buffers, one contiguous piece for rank-major
// [ranks, B, L, H/ranks, D] buffers), while the next layer's kernels run.  No SM is used, nothing
// waits across GPUs inside a kernel, no multicast.
//
// The reference has no counterpart (it runs on one GPU).
#include "common.cuh"

extern "C" int kb200_peer_push(const kb200_push_plan* plan, const void* src_base, size_t offset_bytes,
                               size_t pitch_bytes, size_t width_bytes, size_t rows, void* ready_event,
                               void* compute_stream) {
  using namespace kb200;
  KB_REQUIRE(plan && src_base && ready_event, "peer_push: null pointer");
  KB_REQUIRE(plan->count >= 0 && plan->count <= KB200_MAX_FANOUT, "peer_push: %d peers (0..%d supported)", plan->count,
             KB200_MAX_FANOUT);
  KB_REQUIRE(width_bytes > 0 && width_bytes <= pitch_bytes && offset_bytes + width_bytes <= pitch_bytes,
             "peer_push: a row slice of %zu bytes at offset %zu does not fit a pitch of %zu bytes", width_bytes,
             offset_bytes, pitch_bytes);
  if (rows == 0 || plan->count == 0) return 0;
  // the slice is complete once everything queued on the compute stream so far has run
  KB_CUDA(cudaEventRecord((cudaEvent_t)ready_event, (cudaStream_t)compute_stream));
  const char* src = static_cast<const char*>(src_base) + offset_bytes;
  for (int i = 0; i < plan->count; ++i) {
    KB_REQUIRE(plan->dst[i] && plan->stream[i] && plan->done_event[i], "peer_push: peer %d has a null entry", i);
    cudaStream_t st = (cudaStream_t)plan->stream[i];
    KB_CUDA(cudaStreamWaitEvent(st, (cudaEvent_t)ready_event, 0));
    if (rows == 1)        // one contiguous piece: a plain copy runs at the full link rate, a pitched one does not
      KB_CUDA(cudaMemcpyAsync(static_cast<char*>(plan->dst[i]) + offset_bytes, src, width_bytes, cudaMemcpyDeviceToDevice, st));
    else
      KB_CUDA(cudaMemcpy2DAsync(static_cast<char*>(plan->dst[i]) + offset_bytes, pitch_bytes, src, pitch_bytes,
                                width_bytes, rows, cudaMemcpyDeviceToDevice, st));
    KB_CUDA(cudaEventRecord((cudaEvent_t)plan->done_event[i], st));
  }
  return 0;
}

extern "C" int kb200_stream_wait_events(void* stream, void* const* events, int count) {
  using namespace kb200;
  KB_REQUIRE(count >= 0 && (count == 0 || events), "stream_wait_events: bad arguments");
  for (int i = 0; i < count; ++i)
    if (events[i]) KB_CUDA(cudaStreamWaitEvent((cudaStream_t)stream, (cudaEvent_t)events[i], 0));
  return 0;
}
