"""Generates the golden vectors under tests/golden/ by running the reference project's OWN shader
sources (compiled as C++ into oracle/_ref/libref_attention.so, see oracle/Makefile) on the inputs
its unit tests use, plus two seeded cases that reach the kernels those tests never exercise.

    make -C oracle REF_ROOT=<reference checkout> && python tests/golden/make_golden.py

Needs the reference tree at build time only; the committed .npz files are what the tests read.
Inputs follow the closed forms in the reference's tests:
  flash_kat1  src/ops/flash_attention.rs:242-294   B2 H4 S32 D16, q=k=v=sin(i*0.1)*0.5, causal + full
  flash_kat2  src/ops/flash_attention.rs:297-329   B1 H2 S128 D32, q=k=v=sin(i*0.01)*0.3, causal
  bwd_kat     src/train/helpers.rs:437-494         B2 H4 S16 D8, (i%17)*0.01-0.08 etc., causal
  tiled_seeded   B1 H2 S300 D64 seeded N(0,1): the S>256 online-softmax kernel (flash_attention.metal:45-163)
  decode_seeded  B1 H4 S119 D64 seeded N(0,1): the longest prefix of the greedy-inference pattern
  bwd_seeded     B1 H2 S40 D16 seeded N(0,1): composed backward on random data
  rope_kat       src/ops/rope.rs:128-250: simple (1,2,1,4) i+1; position zero (1,1,2,8) (i+1)*0.1; larger (2,16,4,64)
                 (i%100-50)*0.01; with offset 10 (1,4,2,8) i*0.1 -- rope_f32 outputs, and rope_backward_f32 of
                 the "larger" output; plus one long-position case (1,4,1,128) at offset 8188, seeded
  repeat_kv_kat  src/ops/repeat_kv.rs:308-440: simple (2,4,2->8,4) i; backward (2,4,8->2,4) i*0.1; no repeat
                 (2,4,4,8); roundtrip (1,2,2->4,2) i+1
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import oracle_lib as ol  # noqa: E402
from irontensor_b200 import synth  # noqa: E402


def main():
    assert ol.reference() is not None, "build oracle/_ref first (needs the reference tree)"
    f32 = np.float32

    n = 2 * 4 * 32 * 16
    x = (np.sin((np.arange(n, dtype=f32) * f32(0.1)).astype(f32)) * f32(0.5)).astype(f32).reshape(2, 4, 32, 16)
    np.savez_compressed(os.path.join(HERE, "flash_kat1.npz"), q=x, k=x, v=x,
                        o_causal=ol.ref_fwd(x, x, x, True), o_full=ol.ref_fwd(x, x, x, False))

    n = 1 * 2 * 128 * 32
    x = (np.sin((np.arange(n, dtype=f32) * f32(0.01)).astype(f32)) * f32(0.3)).astype(f32).reshape(1, 2, 128, 32)
    np.savez_compressed(os.path.join(HERE, "flash_kat2.npz"), q=x, k=x, v=x, o_causal=ol.ref_fwd(x, x, x, True))

    n = 2 * 4 * 16 * 8
    i = np.arange(n)
    shp = (2, 4, 16, 8)
    d_o = ((i % 17).astype(f32) * f32(0.01) - f32(0.08)).reshape(shp)
    q = ((i % 13).astype(f32) * f32(0.01) - f32(0.06)).reshape(shp)
    k = ((i % 11).astype(f32) * f32(0.01) - f32(0.05)).reshape(shp)
    v = ((i % 7).astype(f32) * f32(0.01) - f32(0.03)).reshape(shp)
    dq, dk, dv = ol.ref_bwd(q, k, v, d_o)
    np.savez_compressed(os.path.join(HERE, "bwd_kat.npz"), q=q, k=k, v=v, d_o=d_o, dq=dq, dk=dk, dv=dv,
                        o_causal=ol.ref_fwd(q, k, v, True))

    q, k, v = [t.reshape(1, 2, 300, 64) for t in synth.attention_inputs(11, 1, 2, 300, 64, with_do=False)]
    np.savez_compressed(os.path.join(HERE, "tiled_seeded.npz"), seed=11, o_causal=ol.ref_fwd(q, k, v, True),
                        o_full=ol.ref_fwd(q, k, v, False))

    q, k, v = [t.reshape(1, 4, 119, 64) for t in synth.attention_inputs(synth.BASE_SEED + 119, 1, 4, 119, 64, with_do=False)]
    np.savez_compressed(os.path.join(HERE, "decode_seeded.npz"), seed=synth.BASE_SEED + 119, o_causal=ol.ref_fwd(q, k, v, True))

    q, k, v, d_o = [t.reshape(1, 2, 40, 16) for t in synth.attention_inputs(13, 1, 2, 40, 16)]
    dq, dk, dv = ol.ref_bwd(q, k, v, d_o)
    np.savez_compressed(os.path.join(HERE, "bwd_seeded.npz"), seed=13, dq=dq, dk=dk, dv=dv)
    def seq(shape, fn):
        return fn(np.arange(int(np.prod(shape)))).astype(f32).reshape(shape)

    r = {}
    r["simple_in"] = seq((1, 2, 1, 4), lambda i: i.astype(f32) + f32(1.0))
    r["simple_out"] = ol.ref_rope(r["simple_in"], 10000.0, 0)
    r["zero_in"] = seq((1, 1, 2, 8), lambda i: (i.astype(f32) + f32(1.0)) * f32(0.1))
    r["zero_out"] = ol.ref_rope(r["zero_in"], 10000.0, 0)
    r["larger_in"] = seq((2, 16, 4, 64), lambda i: ((i % 100).astype(f32) - f32(50.0)) * f32(0.01))
    r["larger_out"] = ol.ref_rope(r["larger_in"], 10000.0, 0)
    r["larger_back"] = ol.ref_rope(r["larger_out"], 10000.0, 0, inverse=True)
    r["offset_in"] = seq((1, 4, 2, 8), lambda i: i.astype(f32) * f32(0.1))
    r["offset_out"] = ol.ref_rope(r["offset_in"], 10000.0, 10)
    r["long_in"] = synth.attention_inputs(17, 1, 4, 1, 128, with_do=False)[0].reshape(1, 4, 1, 128)
    r["long_out"] = ol.ref_rope(r["long_in"], 10000.0, 8188)
    np.savez_compressed(os.path.join(HERE, "rope_kat.npz"), **r)

    r = {}
    r["simple_in"] = seq((2, 4, 2, 4), lambda i: i.astype(f32))
    r["simple_out"] = ol.ref_repeat_kv(r["simple_in"], 8)
    r["backward_in"] = seq((2, 4, 8, 4), lambda i: i.astype(f32) * f32(0.1))
    r["backward_out"] = ol.ref_repeat_kv(r["backward_in"], 8, backward=True, kv_heads=2)
    r["norepeat_in"] = seq((2, 4, 4, 8), lambda i: i.astype(f32))
    r["norepeat_out"] = ol.ref_repeat_kv(r["norepeat_in"], 4)
    r["roundtrip_in"] = seq((1, 2, 2, 2), lambda i: i.astype(f32) + f32(1.0))
    r["roundtrip_mid"] = ol.ref_repeat_kv(r["roundtrip_in"], 4)
    r["roundtrip_out"] = ol.ref_repeat_kv(r["roundtrip_mid"], 4, backward=True, kv_heads=2)
    np.savez_compressed(os.path.join(HERE, "repeat_kv_kat.npz"), **r)
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    main()
