# Dense, Embedding, Dropout.
# replaces (a::Dense)(x) = NNlib.bias_act!(a.σ, a.weight * xT, a.bias)            src/layers/basic.jl:196-205
function dense_fused(σ, W::B200Matrix{F32}, x::B200Array{F32}, b; save_z::Bool=false)
    out, in = size(W); n = length(x) ÷ in
    y = similar(x, F32, (out, size(x)[2:end]...)); z = save_z ? similar(y) : nothing
    check(ccall(sym(:fb_dense_fwd), Int32, (PV, PV, Int32, Int32, PV, PV, PV, PV, PV, Int64, Int64, Int64),
                fbctx(), fbstream(), act_code(σ), Int32(0), ptr(W), ptr(arr_or_nothing(b)), ptr(x), ptr(y), ptr(z), out, in, n))
    return y, z
end

function (a::Dense{<:Any,<:B200Matrix{F32}})(x::B200Array{F32})
    _size_check(a, x, 1 => size(a.weight, 2))
    first(dense_fused(a.σ, a.weight, x, a.bias))
end

function ChainRulesCore.rrule(::typeof(dense_fused), σ, W::B200Matrix{F32}, x::B200Array{F32}, b; save_z::Bool=false)
    code = act_code(σ)
    y, z = dense_fused(σ, W, x, b; save_z=needs_z(code))
    out, in = size(W); n = length(x) ÷ in
    bb = arr_or_nothing(b)
    function dense_pullback(Δ)
        dy = unthunk(Δ isa Tuple ? Δ[1] : Δ)
        dW = grad_like(W); dx = similar(x)
        db = bb === nothing ? nothing : grad_like(bb)
        delta = code == 0 ? nothing : similar(y)
        check(ccall(sym(:fb_dense_bwd), Int32, (PV, PV, Int32, Int32, PV, PV, PV, PV, PV, PV, PV, PV, PV, Int64, Int64, Int64),
                    fbctx(), fbstream(), code, Int32(0), ptr(W), ptr(x), ptr(y), ptr(z), ptr(dy), ptr(delta), ptr(dW), ptr(db), ptr(dx), out, in, n))
        grad_done!(W); grad_done!(bb)
        return NoTangent(), NoTangent(), dW, dx, db === nothing ? NoTangent() : db
    end
    return (y, z), dense_pullback
end

# The bf16 storage variant (Flux.bf16, src/functor.jl:274): weights, bias, activations and gradients are BFloat16.
const BF16 = B200Arrays.BFloat16Bits       # a 16-bit primitive type holding the raw bf16 pattern
function dense_fused(σ, W::B200Matrix{BF16}, x::B200Array{BF16}, b; save_z::Bool=false)
    out, in = size(W); n = length(x) ÷ in
    y = similar(x, BF16, (out, size(x)[2:end]...)); z = save_z ? similar(y) : nothing
    check(ccall(sym(:fb_dense_fwd_bf16), Int32, (PV, PV, Int32, PV, PV, PV, PV, PV, Int64, Int64, Int64),
                fbctx(), fbstream(), act_code(σ), ptr(W), ptr(arr_or_nothing(b)), ptr(x), ptr(y), ptr(z), out, in, n))
    return y, z
end
function (a::Dense{<:Any,<:B200Matrix{BF16}})(x::B200Array{BF16})
    _size_check(a, x, 1 => size(a.weight, 2))
    first(dense_fused(a.σ, a.weight, x, a.bias))
end
function ChainRulesCore.rrule(::typeof(dense_fused), σ, W::B200Matrix{BF16}, x::B200Array{BF16}, b; save_z::Bool=false)
    code = act_code(σ)
    y, z = dense_fused(σ, W, x, b; save_z=needs_z(code))
    out, in = size(W); n = length(x) ÷ in
    bb = arr_or_nothing(b)
    function dense_bf16_pullback(Δ)
        dy = unthunk(Δ isa Tuple ? Δ[1] : Δ)
        dW = similar(W); dx = similar(x)
        db = bb === nothing ? nothing : similar(bb)
        delta = code == 0 ? nothing : similar(y)
        check(ccall(sym(:fb_dense_bwd_bf16), Int32, (PV, PV, Int32, PV, PV, PV, PV, PV, PV, PV, PV, PV, Int64, Int64, Int64),
                    fbctx(), fbstream(), code, ptr(W), ptr(x), ptr(y), ptr(z), ptr(dy), ptr(delta), ptr(dW), ptr(db), ptr(dx), out, in, n))
        return NoTangent(), NoTangent(), dW, dx, db === nothing ? NoTangent() : db
    end
    return (y, z), dense_bf16_pullback
end
function Flux._to_bf16(x::B200Array{F32})
    y = similar(x, BF16, size(x))
    check(ccall(sym(:fb_cast_f32_bf16), Int32, (PV, PV, PV, PV, Int64), fbctx(), fbstream(), ptr(x), ptr(y), length(x)))
    return y
end
function to_f32(x::B200Array{BF16})
    y = similar(x, F32, size(x))
    check(ccall(sym(:fb_cast_bf16_f32), Int32, (PV, PV, PV, PV, Int64), fbctx(), fbstream(), ptr(x), ptr(y), length(x)))
    return y
end

# ------------------------------------------------------------------------------------------- Embedding ---
# replaces NNlib.gather(m.weight, x) and the padding mask                           src/layers/basic.jl:794-800
function embedding_fused(W::B200Matrix{F32}, idx::B200Array{Int32}, padding_idx::Int32)
    out, vocab = size(W); n = length(idx)
    y = similar(W, F32, (out, size(idx)...))
    check(ccall(sym(:fb_embedding_fwd), Int32, (PV, PV, PV, PV, PV, Int64, Int64, Int64, Int32),
                fbctx(), fbstream(), ptr(W), ptr(idx), ptr(y), out, vocab, n, padding_idx))
    return y
end
(m::Embedding{<:B200Matrix{F32}})(idx::B200Array{Int32}) =
    embedding_fused(m.weight, idx, m.padding_idx === nothing ? Int32(0) : Int32(m.padding_idx))
function ChainRulesCore.rrule(::typeof(embedding_fused), W::B200Matrix{F32}, idx::B200Array{Int32}, padding_idx::Int32)
    out, vocab = size(W); n = length(idx)
    function embedding_pullback(Δ)
        dW = grad_like(W)
        check(ccall(sym(:fb_embedding_bwd), Int32, (PV, PV, PV, PV, PV, Int64, Int64, Int64, Int32),
                    fbctx(), fbstream(), ptr(unthunk(Δ)), ptr(idx), ptr(dW), out, vocab, n, padding_idx))
        grad_done!(W)
        return NoTangent(), dW, NoTangent(), NoTangent()
    end
    return embedding_fused(W, idx, padding_idx), embedding_pullback
end

# --------------------------------------------------------------------------------------------- Dropout ---
# replaces NNlib.dropout(rng, x, p; dims)                                           src/layers/normalise.jl:83
# The mask is a function of (seed, offset, element index); the pullback regenerates it.
const dropout_counter = Ref{UInt64}(0)
function dropout_fused(x::B200Array{F32}, p::Real, seed::UInt64, offset::UInt64)
    y = similar(x)
    check(ccall(sym(:fb_dropout), Int32, (PV, PV, PV, PV, Int64, Float32, UInt64, UInt64),
                fbctx(), fbstream(), ptr(x), ptr(y), length(x), F32(p), seed, offset))
    return y
end
function (d::Dropout)(x::B200Array{F32})
    (_isactive(d, x) && d.p > 0) || return x
    d.dims isa Colon || throw(ArgumentError("Dropout with dims has no B200 kernel"))
    off = dropout_counter[]
    dropout_counter[] += cld(length(x), 4)
    return dropout_fused(x, d.p, UInt64(hash(d.rng) % typemax(UInt64)), off)
end
function ChainRulesCore.rrule(::typeof(dropout_fused), x::B200Array{F32}, p::Real, seed::UInt64, offset::UInt64)
    dropout_pullback(Δ) = (NoTangent(), dropout_fused(unthunk(Δ), p, seed, offset), NoTangent(), NoTangent(), NoTangent())
    return dropout_fused(x, p, seed, offset), dropout_pullback
end
