"""Tiny configurations of the architecture that differ in every size and option.

                    tiny-A        tiny-B         tiny-C
layers              2             3              4 (5 calls: one layer twice,
                                                    one call reads another's cache)
hidden              64            96             80
q heads / kv heads  4 / 2 (GQA)   3 / 1 (MQA)    5 / 5 (MHA)
head_dim            16            32             48 (not hidden / heads)
intermediate        172           256            200
vocabulary          256           97             301
rope_theta          10000         500000         25000
norm eps            1e-5          1e-6           3e-5
output head         tied          untied         untied
positions           384           640            512
window              none          none           40 on two of the layers
norm weights        1             1 + N(0, .1)   1 + N(0, .1)

Two more, small but with the head sizes, group sizes and alignments that the
tensor-core kernels of large models take (tcgen05 / TMA attention for heads of 64
and 128, the tcgen05 GEMM with its fused SwiGLU epilogue and its weight-major
orientation), so that the same four ways of cutting run on those kernels:

                    tiny-D        tiny-E
layers              2             3
hidden              256           320
q heads / kv heads  4 / 2         8 / 2 (groups of 4)
head_dim            64            128 (heads * head_dim = 1024, not hidden)
intermediate        352           464
vocabulary          331           517
rope_theta          10000         500000
norm eps            1e-5          2e-6
output head         untied        tied
positions           768           1024
window              none          150 on the middle layer
norm weights        1 + N(0, .1)  1 + N(0, .1)
"""

TINY_A = dict(architecture="llama_dense", vocab_size=256, d_model=64, n_layers=2, n_heads=4,
              n_kv_heads=2, head_dim=16, intermediate_size=172, max_seq_len=384,
              rope_theta=10000.0, norm_eps=1e-5, tie_embeddings=True)
TINY_B = dict(architecture="llama_dense", vocab_size=97, d_model=96, n_layers=3, n_heads=3,
              n_kv_heads=1, head_dim=32, intermediate_size=256, max_seq_len=640,
              rope_theta=500000.0, norm_eps=1e-6, tie_embeddings=False)
TINY_C = dict(architecture="llama_dense", vocab_size=301, d_model=80, n_layers=4, n_heads=5,
              n_kv_heads=5, head_dim=48, intermediate_size=200, max_seq_len=512,
              rope_theta=25000.0, norm_eps=3e-5, tie_embeddings=False,
              layer_order=[0, 1, 2, 1, 3], cache_source=[None, None, None, None, 2],
              layer_windows=[None, 40, None, 40])

TINY_D = dict(architecture="llama_dense", vocab_size=331, d_model=256, n_layers=2, n_heads=4,
              n_kv_heads=2, head_dim=64, intermediate_size=352, max_seq_len=768,
              rope_theta=10000.0, norm_eps=1e-5, tie_embeddings=False)
TINY_E = dict(architecture="llama_dense", vocab_size=517, d_model=320, n_layers=3, n_heads=8,
              n_kv_heads=2, head_dim=128, intermediate_size=464, max_seq_len=1024,
              rope_theta=500000.0, norm_eps=2e-6, tie_embeddings=True,
              layer_windows=[None, 150, None])

NORM_STD = {"A": 0.0, "B": 0.1, "C": 0.1, "D": 0.1, "E": 0.1}
CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E}


def plain_cfg(d: dict) -> dict:
    """The dict the plain implementation reads (no defaults hidden)."""
    out = dict(d)
    out.setdefault("layer_order", None)
    out.setdefault("cache_source", None)
    out.setdefault("layer_windows", None)
    return out
