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

// Order in which the CTAs of a causal launch are handed out.  A CTA's work grows with its tile index
// rank (0 = most work).  Slice after slice, heaviest tile first, keeps the resident CTAs on two or three
// slices (good for L2) but ends badly: the last slice's heaviest CTA starts when little other work is
// left and the other SMs idle while it runs (3.3 % of the launch at 64 slices x 64 tiles on 148 SMs).
// Taking the slices four at a time and, inside such a group, all rank-0 tiles first, then all rank-1
// tiles, ... brings that tail to 0.4 % and keeps the resident set at four slices.
__device__ inline void grouped_tile_order(int block, int n_tiles, int n_slices, int* slice, int* rank) {
  constexpr int GROUP = 4;
  const int per_group = GROUP * n_tiles;
  const int s0 = (block / per_group) * GROUP;
  const int rem = block % per_group;
  const int gsize = min(GROUP, n_slices - s0);
  *rank = rem / gsize;
  *slice = s0 + rem % gsize;
}

// The same idea for a kernel that is sensitive to how many slices are resident at once (the forward
// streams K/V tiles from L2, and CTAs of one slice share them): slice after slice as long as enough
// slices follow to fill the tail, and only the last eight slices taken together, heaviest tiles first.
// The model gives the same tails as groups of four everywhere (0.4 % at 64 slices, 5 % at 8).
__device__ inline void tail_grouped_order(int block, int n_tiles, int n_slices, int* slice, int* rank) {
  constexpr int TAIL = 8;
  const int head = max(n_slices - TAIL, 0);
  if (block < head * n_tiles) {
    *slice = block / n_tiles;
    *rank = block % n_tiles;
  } else {
    const int rem = block - head * n_tiles;
    const int t = n_slices - head;
    *rank = rem / t;
    *slice = head + rem % t;
  }
}

}  // namespace it
