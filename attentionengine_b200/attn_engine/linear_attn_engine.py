"""LinearAttentionEngine: operator API of the chunked linear-attention / SSD scan
(reference: attention_engine/attn_engine/linear_attn_engine.py:10-52)."""


class LinearAttentionEngine:
    def __init__(self, qkv_meta, q_mod=None, k_mod=None, v_mod=None, decay_mod=None, custom_io=None, tune=False,
                 tune_filename="tune_result", tune_bwd=False):
        raise NotImplementedError("the chunked linear-attention scan kernels are not built yet")
