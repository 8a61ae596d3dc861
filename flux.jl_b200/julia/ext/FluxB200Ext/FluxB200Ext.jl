# ext/FluxB200Ext — Flux package extension for B200 arrays (sits beside ext/FluxCUDAExt.jl).
#
#   Project.toml of Flux gains:   [weakdeps]   B200Arrays = "6f1b7c9e-3b6d-4c57-9a44-b200b200b200"
#                                 [extensions] FluxB200Ext = "B200Arrays"
#
# It adds methods on Flux's own layer call operators, on `Flux.scan`, on `NNlib.dot_product_attention`, on
# `Flux.Losses.logitcrossentropy`, on `Optimisers.apply!` and on the `DistributedUtils.__bcast!/__allreduce!/
# __reduce!` slots for arrays of the new type, plus the ChainRules rrules Zygote needs (Flux defines no rrule for
# its layers; see src/gradient.jl and the NNlib rules it relies on).  `src/` of Flux is not edited.
#
# NOT EXECUTED in this repository's build environment (no Julia toolchain there).  Every ccall below has the
# argument order of include/fluxb200.h; the same entry points are driven from Python by the parity tests.
module FluxB200Ext

using Flux, B200Arrays, ChainRulesCore
using Flux: Dense, LayerNorm, BatchNorm, LSTMCell, GRUCell, _size_check, _isactive
import NNlib, Optimisers
using B200Arrays: B200Array, B200Matrix, B200VecOrMat, check, sym, fbctx, fbstream

const F32 = Float32
const PV = Ptr{Cvoid}
ptr(a::B200Array) = a.ptr
ptr(::Union{Nothing,Bool}) = C_NULL

# activation enum of fluxb200.h; anything else has no kernel and must not fall back to a broadcast
act_code(::typeof(identity)) = Int32(0)
act_code(::typeof(NNlib.relu)) = Int32(1)
act_code(::typeof(tanh)) = Int32(2)
act_code(::typeof(NNlib.tanh_fast)) = Int32(2)
act_code(::typeof(NNlib.sigmoid)) = Int32(3)
act_code(::typeof(NNlib.sigmoid_fast)) = Int32(3)
act_code(::typeof(NNlib.gelu)) = Int32(4)
act_code(f) = throw(ArgumentError("activation $f has no B200 kernel"))
needs_z(code) = code >= 4

# ------------------------------------------------------------------------------------------------ Dense ---
# replaces (a::Dense)(x) = NNlib.bias_act!(a.σ, a.weight * xT, a.bias)            src/layers/basic.jl:196-200
function dense_fused(σ, W::B200Matrix{F32}, x::B200VecOrMat{F32}, b; save_z::Bool=false)
    out, in = size(W); n = size(x, 2)
    y = similar(x, F32, (out, n)); z = save_z ? similar(y) : nothing
    check(ccall(sym(:fb_dense_fwd), Int32, (PV, PV, Int32, Int32, PV, PV, PV, PV, PV, Int64, Int64, Int64),
                fbctx(), fbstream(), act_code(σ), 0, ptr(W), ptr(b), ptr(x), ptr(y), ptr(z), out, in, n))
    return y, z
end

function (a::Dense{<:Any,<:B200Matrix})(x::B200VecOrMat)
    _size_check(a, x, 1 => size(a.weight, 2))
    first(dense_fused(a.σ, a.weight, x, a.bias))
end

function ChainRulesCore.rrule(::typeof(dense_fused), σ, W::B200Matrix{F32}, x::B200VecOrMat{F32}, b)
    code = act_code(σ)
    y, z = dense_fused(σ, W, x, b; save_z=needs_z(code))
    out, in = size(W); n = size(x, 2)
    function dense_pullback(Δ)
        dy = unthunk(Δ isa Tuple ? Δ[1] : Δ)
        dW = similar(W); dx = similar(x)
        db = b isa B200Array ? similar(b) : nothing
        delta = code == 0 ? nothing : similar(y)
        check(ccall(sym(:fb_dense_bwd), Int32, (PV, PV, Int32, Int32, PV, PV, PV, PV, PV, PV, PV, PV, PV, Int64, Int64, Int64),
                    fbctx(), fbstream(), code, 0, ptr(W), ptr(x), ptr(y), ptr(z), ptr(dy), ptr(delta), ptr(dW), ptr(db), ptr(dx), out, in, n))
        return NoTangent(), NoTangent(), dW, dx, db === nothing ? NoTangent() : db
    end
    return (y, z), dense_pullback
end

# ------------------------------------------------------------------------------------------- LayerNorm ---
# replaces a.diag(NNlib.normalise(x; dims=1:length(a.size), eps=a.ϵ))              src/layers/normalise.jl:203-210
function layernorm_fused(a::LayerNorm, x::B200Array{F32})
    d = prod(a.size); n = length(x) ÷ d
    y = similar(x); mean = similar(x, F32, (n,)); rstd = similar(x, F32, (n,))
    γ = a.affine ? a.diag.scale : nothing; β = a.affine ? a.diag.bias : nothing
    check(ccall(sym(:fb_layernorm_fwd), Int32, (PV, PV, PV, PV, PV, PV, PV, PV, Int64, Int64, Float32, Int32),
                fbctx(), fbstream(), ptr(x), ptr(γ), ptr(β), ptr(y), ptr(mean), ptr(rstd), d, n, F32(a.ϵ), act_code(a.λ)))
    return y, mean, rstd
end
(a::LayerNorm)(x::B200Array{F32}) = first(layernorm_fused(a, x))

function ChainRulesCore.rrule(::typeof(layernorm_fused), a::LayerNorm, x::B200Array{F32})
    y, mean, rstd = layernorm_fused(a, x)
    d = prod(a.size); n = length(x) ÷ d
    γ = a.affine ? a.diag.scale : nothing; β = a.affine ? a.diag.bias : nothing
    function layernorm_pullback(Δ)
        dy = unthunk(Δ[1]); dx = similar(x)
        dγ = a.affine ? similar(γ) : nothing; dβ = a.affine ? similar(β) : nothing
        check(ccall(sym(:fb_layernorm_bwd), Int32, (PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, Int64, Int64, Int32),
                    fbctx(), fbstream(), ptr(x), ptr(γ), ptr(β), ptr(mean), ptr(rstd), ptr(dy), ptr(dx), ptr(dγ), ptr(dβ), d, n, act_code(a.λ)))
        da = a.affine ? Tangent{typeof(a)}(; diag=Tangent{typeof(a.diag)}(; scale=dγ, bias=dβ)) : NoTangent()
        return NoTangent(), da, dx
    end
    return (y, mean, rstd), layernorm_pullback
end

# ------------------------------------------------------------------------------------------- BatchNorm ---
# replaces NNlib.batchnorm(γ, β, x, μ, σ², momentum; eps, training, track_stats) then BN.λ.(y)   normalise.jl:292-304
function (BN::BatchNorm)(x::B200Array{F32,N}) where {N}
    _size_check(BN, x, N - 1 => BN.chs)
    training = _isactive(BN, x)
    c = BN.chs; n = size(x, N); s = length(x) ÷ (c * n)
    if training === true && s * n == 1
        throw(ArgumentError("BatchNorm expected more than 1 value per channel when training, got input of size $(size(x))."))
    end
    y = similar(x)
    if training === true || !BN.track_stats
        mean = similar(x, F32, (c,)); rstd = similar(x, F32, (c,))
        check(ccall(sym(:fb_batchnorm_fwd_train), Int32, (PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, Int64, Int64, Int64, Float32, Float32, Int32, Int32),
                    fbctx(), fbstream(), ptr(x), ptr(BN.γ), ptr(BN.β), ptr(BN.μ), ptr(BN.σ²), ptr(y), ptr(mean), ptr(rstd), s, c, n,
                    F32(BN.ϵ), F32(BN.momentum), act_code(BN.λ), Int32(training === true && BN.track_stats)))
    else
        check(ccall(sym(:fb_batchnorm_fwd_infer), Int32, (PV, PV, PV, PV, PV, PV, PV, PV, Int64, Int64, Int64, Float32, Int32),
                    fbctx(), fbstream(), ptr(x), ptr(BN.γ), ptr(BN.β), ptr(BN.μ), ptr(BN.σ²), ptr(y), s, c, n, F32(BN.ϵ), act_code(BN.λ)))
    end
    return y
end
# (the rrule calls fb_batchnorm_bwd with the saved mean / rstd, same shape as the LayerNorm rule above)

# ------------------------------------------------------------------------------------------ Recurrence ---
# replaces scan(cell, x, state): the host loop over eachslice(x, dims=2)          src/layers/recurrent.jl:1-8
function Flux.scan(cell::LSTMCell{<:B200Matrix}, x::B200Array{F32,3}, (h0, c0))
    in, T, B = size(x); H = size(cell.Wh, 2)
    out = similar(x, F32, (H, T, B)); hT = similar(x, F32, (H, B)); cT = similar(hT)
    b = cell.bias isa B200Array ? cell.bias : nothing
    check(ccall(sym(:fb_lstm_fwd), Int32, (PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, Int64, Int64, Int64, Int64),
                fbctx(), fbstream(), ptr(cell.Wi), ptr(cell.Wh), ptr(b), ptr(x), C_NULL, C_NULL, ptr(out), ptr(hT), ptr(cT), C_NULL, in, H, T, B))
    return out, (hT, cT)
end
# GRUCell: the same with fb_gru_fwd; the rrules allocate the cache (fb_lstm_cache_bytes / fb_gru_cache_bytes)
# and call fb_lstm_bwd / fb_gru_bwd.

# ------------------------------------------------------------------------------------------- attention ---
# replaces NNlib.dot_product_attention(q, k, v, bias; nheads, mask, fdrop)         src/layers/attention.jl:128
function NNlib.dot_product_attention(q::B200Array{F32,3}, k::B200Array{F32,3}, v::B200Array{F32,3}, bias=nothing;
                                     nheads::Int=1, mask=nothing, fdrop=identity)
    bias === nothing || throw(ArgumentError("additive attention bias has no B200 kernel"))
    E, Lq, B = size(q); Ev, Lk, _ = size(v)
    causal = mask isa NNlib.AbstractMask ? 1 : 0     # a lazy causal mask; a Bool matrix is passed as UInt8 [Lk, Lq]
    o = similar(q, F32, (Ev, Lq, B)); lse = similar(q, F32, (Lq, nheads, B))
    check(ccall(sym(:fb_attn_fwd), Int32, (PV, PV, PV, PV, PV, PV, PV, PV, Int64, Int64, Int64, Int64, Int64, Int32, Int32),
                fbctx(), fbstream(), ptr(q), ptr(k), ptr(v), C_NULL, ptr(o), ptr(lse), E, Ev, Lq, Lk, B, nheads, causal))
    return o, LazyScores(q, k, lse, nheads, causal)   # α materialises through fb_attn_scores on first use
end
struct LazyScores; q; k; lse; nheads; causal; end

# ------------------------------------------------------------------------------------------------- loss ---
# replaces mean(.-sum(y .* logsoftmax(ŷ; dims=1); dims=1))                         src/losses/functions.jl:270-273
function Flux.Losses.logitcrossentropy(ŷ::B200Matrix{F32}, y::B200Matrix{F32}; dims=1, agg=Flux.mean)
    c, n = size(ŷ); loss = similar(ŷ, F32, (1,))
    check(ccall(sym(:fb_logitcrossentropy_dense), Int32, (PV, PV, PV, PV, PV, PV, Int64, Int64, Float32),
                fbctx(), fbstream(), ptr(ŷ), ptr(y), ptr(loss), C_NULL, c, n, 1f0))
    return Array(loss)[1]
end

# ------------------------------------------------------------------------------------------- optimiser ---
# replaces the per-leaf broadcasts of Optimisers.apply!(::Adam, ...) and `x .-= dx`   src/train.jl:425
Optimisers.maywrite(::B200Array) = true
function Optimisers.apply!(o::Optimisers.Adam, (m, v, βt), x::B200Array{F32}, dx::B200Array{F32})
    ws = [x.ptr]; gs = [dx.ptr]; ms = [m.ptr]; vs = [v.ptr]; ns = Int64[length(x)]
    check(ccall(sym(:fb_adam_step), Int32, (PV, PV, Int32, Ptr{PV}, Ptr{PV}, Ptr{PV}, Ptr{PV}, Ptr{Int64}, Float32, Float32, Float32, Float32, Float32, Float32, Float32),
                fbctx(), fbstream(), 1, ws, gs, ms, vs, ns, F32(o.eta), F32(o.beta[1]), F32(o.beta[2]), F32(o.epsilon), F32(βt[1]), F32(βt[2]), 1f0))
    return (m, v, βt .* o.beta), Optimisers.Zero()       # the kernel already subtracted the step from x
end

# ----------------------------------------------------------------------------------- DistributedUtils ---
# replaces NCCL.Allreduce! / Broadcast! / Reduce! on CuArray                       ext/FluxMPINCCLExt/FluxMPINCCLExt.jl:38-107
const DU = Flux.DistributedUtils
const comm = Ref{PV}(C_NULL)      # created by fb_comm_init_rank after the MPI broadcast of the unique id (FluxMPINCCLExt.jl:19-30)
opcode(::typeof(+)) = Int32(0)
opcode(::typeof(DU.avg)) = Int32(1)
function DU.__allreduce!(::DU.NCCLBackend, buf::B200Array{F32}, op::F, ::B200Device) where {F}
    check(ccall(sym(:fb_allreduce), Int32, (PV, PV, PV, PV, Int64, Int32), comm[], fbstream(), ptr(buf), ptr(buf), length(buf), opcode(op)))
    return buf
end
function DU.__bcast!(::DU.NCCLBackend, buf::B200Array{F32}, ::B200Device; root=0)
    check(ccall(sym(:fb_bcast), Int32, (PV, PV, PV, PV, Int64, Int32), comm[], fbstream(), ptr(buf), ptr(buf), length(buf), Int32(root)))
    return buf
end
function DU.__reduce!(::DU.NCCLBackend, buf::B200Array{F32}, op::F, ::B200Device; root=0) where {F}
    check(ccall(sym(:fb_reduce), Int32, (PV, PV, PV, PV, Int64, Int32, Int32), comm[], fbstream(), ptr(buf), ptr(buf), length(buf), opcode(op), Int32(root)))
    return buf
end

# Bucketed, overlapped gradient averaging for DistributedOptimizer                  src/distributed/public_api.jl:286-300
# Gradients of a model moved to the device live in ONE flat buffer (GradientArena); every leaf's gradient is a view
# into it, registered with the native bucket set.  The rrules above write dW / db straight into those views and call
# `mark_ready!`; a bucket's mean all-reduce starts on the library's communication stream as soon as its last leaf is
# ready, while the reverse sweep goes on.  `apply!` of the wrapped rule then only waits for the buckets.
mutable struct GradientArena
    flat::B200Array{F32,1}
    set::PV                          # fb_bucket_set*
    leaf_id::IdDict{Any,Int32}       # parameter array => leaf id
    view::IdDict{Any,B200Array}      # parameter array => its gradient view
end
const arena = Ref{Union{Nothing,GradientArena}}(nothing)

function GradientArena(params::Vector; bucket_bytes::Int = 64 << 20)
    pad(n) = cld(n, 64) * 64                               # every slice starts on a 256-byte boundary
    total = sum(pad(length(p)) for p in params)
    flat = B200Arrays.zeros(F32, total)
    ends = Int64[]; off = 0; start = 0
    offs = Dict{Any,Int}()
    for p in reverse(params)                               # the order the reverse sweep produces gradients in
        offs[p] = off; off += pad(length(p))
        if (off - start) * 4 >= bucket_bytes; push!(ends, off); start = off; end
    end
    (isempty(ends) || ends[end] != total) && push!(ends, total)
    set = Ref{PV}(C_NULL)
    check(ccall(sym(:fb_bucket_create), Int32, (PV, PV, PV, Int64, Int32, Ptr{Int64}, PV, Ptr{PV}),
                fbctx(), comm[], ptr(flat), total, Int32(length(ends)), ends, C_NULL, set))
    a = GradientArena(flat, set[], IdDict{Any,Int32}(), IdDict{Any,B200Array}())
    for p in params
        id = Ref{Int32}(-1)
        check(ccall(sym(:fb_bucket_register), Int32, (PV, Int64, Int64, Ptr{Int32}), a.set, offs[p], length(p), id))
        a.leaf_id[p] = id[]
        a.view[p] = B200Arrays.view1d(flat, offs[p], size(p))
    end
    return a
end
begin_step!(a::GradientArena) = check(ccall(sym(:fb_bucket_begin_step), Int32, (PV,), a.set))
mark_ready!(a::GradientArena, p) = check(ccall(sym(:fb_bucket_mark_ready), Int32, (PV, Int32, PV), a.set, a.leaf_id[p], fbstream()))
wait_all!(a::GradientArena) = check(ccall(sym(:fb_bucket_wait), Int32, (PV, PV), a.set, fbstream()))

function Optimisers.apply!(o::DU.DistributedOptimizer{<:DU.NCCLBackend}, state, x::B200Array{F32}, dx::B200Array{F32})
    a = arena[]
    if a !== nothing && haskey(a.view, x) && ptr(a.view[x]) == ptr(dx)
        wait_all!(a)                                       # averaged in its bucket already: do not reduce twice
    else
        DU.allreduce!(o.backend, dx, DU.avg)
    end
    return Optimisers.apply!(o.opt, state, x, dx)
end

# --------------------------------------------------------------------------------------------- bf16 ---
# Flux.bf16 on the device: parameters keep BFloat16 VALUES in Float32 storage (rounding bit-exact with _to_bf16,
# src/functor.jl:161-166); Dense then multiplies with the single TF32 pass (exact products, Float32 accumulation).
function Flux._to_bf16(x::B200Array{F32})
    y = similar(x)
    check(ccall(sym(:fb_round_bf16), Int32, (PV, PV, PV, PV, Int64), fbctx(), fbstream(), ptr(x), ptr(y), length(x)))
    return y
end

end # module
