"""irontensor_b200: the B200 (sm_100a) attention path for the IronTensor library.

Host-side mirror of the reference's attention interface (`flash_attention`, `attention`,
`attention_backward_recompute`, `Tensor`, `CommandBatch`) over the C ABI declared in
include/irontensor_b200.h.  Importing this package does not need a GPU; using it does."""
from .ops import (CommandBatch, Precision, Tensor, attention, attention_backward, attention_backward_recompute, attention_gqa,
                  attention_gqa_backward, attention_decode, attention_packed, attention_packed_backward, linear_backward, linear_forward, qkv_rope_forward, rope,
                  rope_qk,  # noqa: F401
                  flash_attention, context, raw, HostAttentionStep)
