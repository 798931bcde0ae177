// Where a [batch, heads, seq, head_dim] element lives.  Both the reference's flash-attention layout
// [B,H,S,D] (src/ops/flash_attention.rs:65-70) and its attention() layout [B,S,H,D]
// (src/ops/attention.rs:279-285) are described by three strides, in elements; the kernels take the
// strides, so neither layout needs the transposes the reference runs around its attention
// (src/ops/transpose.rs:277-395, called at src/train/forward.rs:125-127,141).
#pragma once

namespace it {

// Grouped-query attention (the reference expands K/V with repeat_kv, src/shaders/repeat_kv.metal:19-47):
// a K/V tensor with heads/group heads is described with `heads` = the number of QUERY heads and
// `group` = query heads per K/V head, so that slice(query slice index) lands on the K/V head that
// query head reads and no expanded copy is ever made.
struct TensorStrides {
  long long row;     // between consecutive sequence positions of one head
  long long head;    // between heads of one batch entry
  long long batch;   // between batch entries
  int heads;         // query heads: the slice index is batch * heads + head
  int group = 1;     // query heads per head of this tensor (1 for Q, O and their gradients)
  __host__ __device__ long long slice(int bh) const { return (bh / heads) * batch + ((bh % heads) / group) * head; }
};

}  // namespace it
