"""The reference's example programs written against this package: the OnlineFunc definitions and engine
factories of attn_script/mha.py, gqa.py, sigmoidattn.py, reluattn.py, retention.py, mla_decode.py,
gqa_inference.py and mamba2_ngroup1.py, plus seeded input generators with the benchmark's distributions.
The benchmark, the build step and the tests all take their engines from here."""
import math

import torch

from .attn_engine import AttentionEngine, LinearAttentionEngine, OnlineFunc
from .core import CustomIO, SymbolScalar, Var, meta_tensor


class OnlineSoftmax(OnlineFunc):
    """attn_script/mha.py:27-84."""

    def __init__(self):
        super().__init__({"m": SymbolScalar("m", Var("-inf")), "r": SymbolScalar("r", Var("0.0"))},
                         {"lse": SymbolScalar("lse", Var("0.0"))}, CustomIO())

    @staticmethod
    def online_fwd(scores, online_rowscales, b, h, q_idx):
        m, r = online_rowscales["m"], online_rowscales["r"]
        m_new = m.max(scores.get_reduce("max"))
        scale_tmp = (m - m_new).exp()
        r = r * scale_tmp
        scores = (scores - m_new).exp()
        r = r + scores.get_reduce("sum")
        return scores, {"m": m_new, "r": r}, scale_tmp

    @staticmethod
    def online_fwd_epilogue(o, online_rowscales, b, h, q_idx):
        o_new = o / online_rowscales["r"]
        lse = (online_rowscales["r"]).log() + online_rowscales["m"]
        return o_new, {"lse": lse}

    @staticmethod
    def forward(scores, final_rowscales, b, h, q_idx, kv_idx):
        return (scores - final_rowscales["lse"]).exp()

    @staticmethod
    def backward(dp, scores, final_rowscales, doosum_rowscales, b, h, q_idx, kv_idx):
        return (dp - doosum_rowscales) * scores


class OnlineIdentity(OnlineFunc):
    """attn_script/sigmoidattn.py:24-49, reluattn.py:21-46."""

    def __init__(self):
        super().__init__({}, {}, CustomIO())

    @staticmethod
    def online_fwd(scores, online_rowscales, b, h, q_idx):
        return scores, online_rowscales, SymbolScalar("o_scale", Var("1"))

    @staticmethod
    def online_fwd_epilogue(o, online_rowscales, b, h, q_idx):
        return o, {}

    @staticmethod
    def forward(scores, final_rowscales, b, h, q_idx, kv_idx):
        return scores

    @staticmethod
    def backward(dp, scores, final_rowscales, doosum_rowscales, b, h, q_idx, kv_idx):
        return dp


def causal_mask(b, h, q_idx, kv_idx):
    return q_idx >= kv_idx


def metas(B, Hq, Hkv, S, D, DV, dtype):
    return (meta_tensor(B, Hq, S, D, dtype=dtype), meta_tensor(B, Hkv, S, D, dtype=dtype),
            meta_tensor(B, Hkv, S, DV, dtype=dtype))


class OnlineSoftmaxSplit(OnlineSoftmax):
    """Online softmax with the split-KV merge of attn_script/gqa_inference.py:72-80 / mla_decode.py."""

    @staticmethod
    def combine(final_rowscales):
        lse = final_rowscales["lse"]
        lse_max = lse.get_reduce("max")
        row_sum = (lse - lse_max).exp()
        row_sum_sum = row_sum.get_reduce("sum")
        lse_sum = row_sum_sum.log() + lse_max
        return (lse - lse_sum).exp()


def decode_engine(B, Hq, Hkv, Sq, Skv, D, dtype, scale=None, online=None):
    """q_len != kv_len: the split-KV decode path (reference scripts gqa_inference.py / mha_inference.py)."""
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    metas_ = (meta_tensor(B, Hq, Sq, D, dtype=dtype), meta_tensor(B, Hkv, Skv, D, dtype=dtype),
              meta_tensor(B, Hkv, Skv, D, dtype=dtype))
    return AttentionEngine(metas_, CustomIO({}), score_mod=lambda s, c, b, h, q, kv: s * scale, mask_mod=None,
                           online_func=online if online is not None else OnlineSoftmaxSplit())


def softmax_engine(B, Hq, Hkv, S, D, DV, dtype, causal, scale=None, **kw):
    scale = 1.0 / math.sqrt(D) if scale is None else scale

    def score_mod(score, custom_fwd_inputs, b, h, q_idx, kv_idx):
        return score * scale

    return AttentionEngine(metas(B, Hq, Hkv, S, D, DV, dtype), CustomIO({}), score_mod=score_mod,
                           mask_mod=causal_mask if causal else None, online_func=OnlineSoftmax(), **kw)


def sigmoid_engine(B, H, S, D, dtype, causal, scale=None):
    """P = sigmoid(score * scale + bias) in the reference's tanh form (attn_script/sigmoidattn.py:14-18);
    bias arrives as the custom input ``softmax_bias`` of shape (1,)."""
    scale = 1.0 / math.sqrt(D) if scale is None else scale

    def score_mod(score, custom_fwd_inputs, b, h, q_idx, kv_idx):
        softmax_bias = custom_fwd_inputs.input_tensors["softmax_bias"]
        score = score * scale + softmax_bias
        return ((score * 0.5).tanh() + 1) * 0.5

    return AttentionEngine(metas(B, H, H, S, D, D, dtype), CustomIO({"softmax_bias": (1,)}), score_mod=score_mod,
                           mask_mod=causal_mask if causal else None, online_func=OnlineIdentity())


def relu_engine(B, H, S, D, dtype, causal=False, scale=None, post_scale=1.0):
    """P = relu(score * scale) * post_scale (attn_script/reluattn.py:14-17)."""
    scale = 1.0 / math.sqrt(D) if scale is None else scale

    def score_mod(score, custom_fwd_inputs, b, h, q_idx, kv_idx):
        score = (score * scale).max(0)
        return score * post_scale if post_scale != 1.0 else score

    return AttentionEngine(metas(B, H, H, S, D, D, dtype), CustomIO({}), score_mod=score_mod,
                           mask_mod=causal_mask if causal else None, online_func=OnlineIdentity())


def seeded_qkv(B, Hq, Hkv, S, D, DV, dtype, seed=0, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, S, Hq, D, generator=g).to(dtype)
    k = torch.randn(B, S, Hkv, D, generator=g).to(dtype)
    v = torch.randn(B, S, Hkv, DV, generator=g).to(dtype)
    d_o = torch.randn(B, S, Hq, DV, generator=g).to(dtype)
    return [t.to(device) for t in (q, k, v, d_o)]


def mla_engine(B, H, S, dtype, scale):
    """attn_script/mla_decode.py:88-118 with the scale chosen by the caller's score_mod."""
    def score_mod(score, custom_fwd_inputs, b, h, q_idx, kv_idx):
        return score * scale

    qkv = (meta_tensor(B, H, 1, 576, dtype=dtype), meta_tensor(B, 1, S, 576, dtype=dtype),
           meta_tensor(B, 1, S, 512, dtype=dtype))
    return AttentionEngine(qkv, CustomIO({}), score_mod=score_mod, mask_mod=None, online_func=OnlineSoftmaxSplit(),
                           kv_shared=True)


def mamba2_engine(B, H, T, DK, DV, dtype, d_skip=False):
    """attn_script/mamba2_ngroup1.py:26-63: decay_mod = decay * A, v_mod = v * dt, one q / k head (ngroups = 1).
    ``d_skip``: add the benchmark configuration's skip connection o += D[h] * x as an ``o_mod`` over a fourth custom
    input D [1, heads] (the reference's harness runs without it, benchmark/bench_utils.py:304-308)."""
    def decay_mod(decay, custom_io):
        return decay * custom_io.input_tensors["A"]

    def v_mod(v, custom_io):
        return v * custom_io.input_tensors["dt"]

    def o_mod(o, v, custom_io):
        return o + v * custom_io.input_tensors["D"]

    metas_ = (meta_tensor(B, 1, T, DK, dtype=dtype), meta_tensor(B, 1, T, DK, dtype=dtype), meta_tensor(B, H, T, DV, dtype=dtype))
    customs = {"A": (1, "heads"), "dt": ("batch", "heads", "seq_len")}
    if d_skip:
        customs["D"] = (1, "heads")
    return LinearAttentionEngine(metas_, decay_mod=decay_mod, v_mod=v_mod, custom_io=CustomIO(customs),
                                 o_mod=o_mod if d_skip else None)


def mamba2_inputs(B, H, T, DK, DV, dtype, seed=0):
    """The benchmark's distributions: x, B, C ~ N(0,1); dt = softplus(N(0,1) - 4); A = -exp(U(ln 1, ln 16))."""
    import math
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, H, T, DV, generator=g).to(dtype)
    Bm = torch.randn(B, 1, T, DK, generator=g).to(dtype)
    Cm = torch.randn(B, 1, T, DK, generator=g).to(dtype)
    dt = torch.nn.functional.softplus(torch.randn(B, H, T, generator=g) - 4.0)
    A = -torch.exp(torch.rand(H, generator=g) * math.log(16.0))
    return x, dt, A, Bm, Cm


class OnlineRetention(OnlineFunc):
    """Row normaliser max(sum |score|, 1), the recurrence of attn_script/retention.py:19-71."""

    def __init__(self):
        super().__init__({"r_wo_clamp": SymbolScalar("r_wo_clamp", Var("0.0")), "r": SymbolScalar("r", Var("0.0"))},
                         {"r": SymbolScalar("r", Var("0.0"))}, CustomIO())

    @staticmethod
    def online_fwd(scores, online_rowscales, b, h, q_idx):
        r_wo_clamp = online_rowscales["r_wo_clamp"] + scores.get_reduce("abssum")
        r_new = r_wo_clamp.max(1.0)
        o_scale = online_rowscales["r"] / r_new
        return scores / r_new, {"r_wo_clamp": r_wo_clamp, "r": r_new}, o_scale

    @staticmethod
    def online_fwd_epilogue(o, online_rowscales, b, h, q_idx):
        return o, {"r": online_rowscales["r"]}

    @staticmethod
    def forward(scores, final_rowscales, b, h, q_idx, kv_idx):
        return scores / final_rowscales["r"]

    @staticmethod
    def backward(dp, scores, final_rowscales, doosum_rowscales, b, h, q_idx, kv_idx):
        return dp / final_rowscales["r"]


def retention_engine(B, H, S, D, DV, dtype):
    """Parallel retention (attn_script/retention.py:14-17, 93-104): the decay mask is a tile-shaped custom input
    [1, heads, seq_len, seq_len_kv] multiplied into the scores; causal mask with additive mask value 0."""

    def score_mod(score, custom_fwd_inputs, b, h, q_idx, kv_idx):
        return score * custom_fwd_inputs.input_tensors["mask"]

    return AttentionEngine(metas(B, H, H, S, D, DV, dtype), CustomIO({"mask": (1, "heads", "seq_len", "seq_len_kv")}),
                           score_mod=score_mod, mask_mod=causal_mask, online_func=OnlineRetention(), mask_value="0")
