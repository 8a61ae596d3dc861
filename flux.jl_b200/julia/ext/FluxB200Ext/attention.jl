# Attention.
# replaces NNlib.dot_product_attention(q, k, v, bias; nheads, mask, fdrop)         src/layers/attention.jl:128
#
# mask: `nothing`, a Bool matrix [kv_len, q_len] (true = keep), or `CausalMask()`.  NNlib.make_causal_mask returns a
# plain Bool matrix; a square upper-triangular one is recognised by value (one pass on the host, it is tiny compared
# with the attention itself) so that the kernel can skip the masked key blocks instead of reading a mask.
struct CausalMask end
is_causal(m::AbstractMatrix{Bool}) = size(m, 1) == size(m, 2) && all(m[j, i] == (j <= i) for i in axes(m, 2), j in axes(m, 1))
is_causal(::CausalMask) = true
is_causal(::Any) = false

struct LazyScores      # the second return value α[kv, q, heads, batch], computed on first use
    q; k; lse; mask; nheads::Int; causal::Bool
end
function materialize(s::LazyScores)
    E, Lq, B = size(s.q); Lk = size(s.k, 2)
    α = similar(s.q, F32, (Lk, Lq, s.nheads, B))
    check(ccall(sym(:fb_attn_scores), Int32, (PV, PV, PV, PV, PV, PV, PV, Int64, Int64, Int64, Int64, Int32, Int32),
                fbctx(), fbstream(), ptr(s.q), ptr(s.k), ptr(s.mask), ptr(s.lse), ptr(α), E, Lq, Lk, B, Int32(s.nheads), Int32(s.causal)))
    return α
end
Base.Array(s::LazyScores) = Array(materialize(s))
Base.size(s::LazyScores) = (size(s.k, 2), size(s.q, 2), s.nheads, size(s.q, 3))

function attention_fused(q::B200Array{F32,3}, k::B200Array{F32,3}, v::B200Array{F32,3}, mask, nheads::Int)
    E, Lq, B = size(q); Ev, Lk, _ = size(v)
    (E % nheads == 0 && Ev % nheads == 0) || throw(ArgumentError("qk_dim = $E and v_dim = $Ev should be divisible by nheads = $nheads"))
    causal = is_causal(mask)
    m8 = (mask === nothing || causal) ? nothing : B200Array(UInt8.(mask))      # [kv_len, q_len], nonzero = keep
    m8 === nothing || size(m8) == (Lk, Lq) || throw(DimensionMismatch("mask of size $(size(m8)) must be (kv_len, q_len) = ($Lk, $Lq)"))
    o = similar(q, F32, (Ev, Lq, B)); lse = similar(q, F32, (Lq, nheads, B))
    check(ccall(sym(:fb_attn_fwd), Int32, (PV, PV, PV, PV, PV, PV, PV, PV, Int64, Int64, Int64, Int64, Int64, Int32, Int32),
                fbctx(), fbstream(), ptr(q), ptr(k), ptr(v), ptr(m8), ptr(o), ptr(lse), E, Ev, Lq, Lk, B, Int32(nheads), Int32(causal)))
    return o, lse, m8, causal
end

function NNlib.dot_product_attention(q::B200Array{F32,3}, k::B200Array{F32,3}, v::B200Array{F32,3}, bias=nothing;
                                     nheads::Int=1, mask=nothing, fdrop=identity)
    bias === nothing || throw(ArgumentError("additive attention bias has no B200 kernel; pass a boolean mask"))
    (fdrop === identity || (fdrop isa Dropout && fdrop.p == 0)) ||
        throw(ArgumentError("dropout on the attention weights has no B200 kernel (they are never materialised); use dropout_prob = 0"))
    o, lse, m8, causal = attention_fused(q, k, v, mask, nheads)
    return o, LazyScores(q, k, lse, m8, nheads, causal)
end

function ChainRulesCore.rrule(::typeof(attention_fused), q::B200Array{F32,3}, k::B200Array{F32,3}, v::B200Array{F32,3}, mask, nheads::Int)
    o, lse, m8, causal = attention_fused(q, k, v, mask, nheads)
    E, Lq, B = size(q); Ev, Lk, _ = size(v)
    function attention_pullback(Δ)
        dout = unthunk(Δ[1])
        dq = similar(q); dk = similar(k); dv = similar(v)
        check(ccall(sym(:fb_attn_bwd), Int32, (PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, Int64, Int64, Int64, Int64, Int64, Int32, Int32),
                    fbctx(), fbstream(), ptr(q), ptr(k), ptr(v), ptr(m8), ptr(o), ptr(lse), ptr(dout), ptr(dq), ptr(dk), ptr(dv),
                    E, Ev, Lq, Lk, B, Int32(nheads), Int32(causal)))
        return NoTangent(), dq, dk, dv, NoTangent(), NoTangent()
    end
    return (o, lse, m8, causal), attention_pullback
end
# The attention weights carry no cotangent path: a loss that reads α (test/layers/attention.jl:56-61) must materialise
# it and is then outside what this extension differentiates; `first ∘ mha` (test/test_module.jl:63) is the supported form.
ChainRulesCore.@non_differentiable materialize(::LazyScores)
