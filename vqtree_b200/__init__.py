"""B200-native fused vector-quantised attention (the hot path of LouChao98/vqtree).

``vqtree_b200.native``  ctypes binding of the C ABI in ``include/vqattn.h`` (libvqattn.so).
``vqtree_b200.api``     tensor-level entry points (assign, aggregates, prefill, decode).
``vqtree_b200.mini_vq``, ``fused_vq_attn``, ``fused_local_attn_rerope``, ``attn_vq``
                        mirrors of the reference's call signatures for this path.
"""
__all__ = ["native", "api"]
