# LayerNorm, BatchNorm, GroupNorm, InstanceNorm.
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
        dγ = grad_like(γ); dβ = grad_like(β)
        check(ccall(sym(:fb_layernorm_bwd), Int32, (PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, Int64, Int64, Int32),
                    fbctx(), fbstream(), ptr(x), ptr(γ), ptr(β), ptr(mean), ptr(rstd), ptr(dy), ptr(dx), ptr(dγ), ptr(dβ), d, n, act_code(a.λ)))
        grad_done!(γ); grad_done!(β)
        da = a.affine ? Tangent{typeof(a)}(; diag=Tangent{typeof(a.diag)}(; scale=dγ, bias=dβ)) : NoTangent()
        return NoTangent(), da, dx
    end
    return (y, mean, rstd), layernorm_pullback
end

# replaces NNlib.batchnorm(γ, β, x, μ, σ², momentum; eps, training, track_stats) then BN.λ.(y)   normalise.jl:292-304
# Returns (y, mean, rstd); mean / rstd are `nothing` on the inference path.
function batchnorm_fused(BN::BatchNorm, x::B200Array{F32,N}, training::Bool) where {N}
    c = BN.chs; n = size(x, N); s = length(x) ÷ (c * n)
    if training && s * n == 1
        throw(ArgumentError("BatchNorm expected more than 1 value per channel when training, got input of size $(size(x)). " *
                            "The batch variance of a single value is undefined; use a larger batch or call `testmode!` for inference."))
    end
    y = similar(x)
    if training || !BN.track_stats
        mean = similar(x, F32, (c,)); rstd = similar(x, F32, (c,))
        check(ccall(sym(:fb_batchnorm_fwd_train), Int32, (PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, Int64, Int64, Int64, Float32, Float32, Int32, Int32),
                    fbctx(), fbstream(), ptr(x), ptr(BN.γ), ptr(BN.β), ptr(BN.μ), ptr(BN.σ²), ptr(y), ptr(mean), ptr(rstd), s, c, n,
                    F32(BN.ϵ), F32(BN.momentum), act_code(BN.λ), Int32(training && BN.track_stats)))
        return y, mean, rstd
    end
    check(ccall(sym(:fb_batchnorm_fwd_infer), Int32, (PV, PV, PV, PV, PV, PV, PV, PV, Int64, Int64, Int64, Float32, Int32),
                fbctx(), fbstream(), ptr(x), ptr(BN.γ), ptr(BN.β), ptr(BN.μ), ptr(BN.σ²), ptr(y), s, c, n, F32(BN.ϵ), act_code(BN.λ)))
    return y, nothing, nothing
end
function (BN::BatchNorm)(x::B200Array{F32,N}) where {N}
    _size_check(BN, x, N - 1 => BN.chs)
    first(batchnorm_fused(BN, x, _isactive(BN, x) === true))
end
function ChainRulesCore.rrule(::typeof(batchnorm_fused), BN::BatchNorm, x::B200Array{F32,N}, training::Bool) where {N}
    y, mean, rstd = batchnorm_fused(BN, x, training)
    c = BN.chs; n = size(x, N); s = length(x) ÷ (c * n)
    function batchnorm_pullback(Δ)
        mean === nothing && throw(ArgumentError("BatchNorm in test mode with tracked statistics is differentiated through fb_batchnorm_fwd_infer only as a constant; call trainmode!"))
        dy = unthunk(Δ[1]); dx = similar(x)
        dγ = BN.affine ? grad_like(BN.γ) : nothing; dβ = BN.affine ? grad_like(BN.β) : nothing
        check(ccall(sym(:fb_batchnorm_bwd), Int32, (PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, Int64, Int64, Int64, Int32),
                    fbctx(), fbstream(), ptr(x), ptr(BN.γ), ptr(BN.β), ptr(mean), ptr(rstd), ptr(dy), ptr(dx), ptr(dγ), ptr(dβ), s, c, n, act_code(BN.λ)))
        BN.affine && (grad_done!(BN.γ); grad_done!(BN.β))
        dBN = BN.affine ? Tangent{typeof(BN)}(; γ=dγ, β=dβ) : NoTangent()
        return NoTangent(), dBN, dx, NoTangent()
    end
    return (y, mean, rstd), batchnorm_pullback
end

# replaces NNlib.groupnorm(γ, β, x, G; eps) / NNlib.instancenorm(...)              normalise.jl:388-393, 486-489
function groupnorm_fused(γ, β, x::B200Array{F32,N}, G::Int, ϵ, λ) where {N}
    c = size(x, N - 1); n = size(x, N); s = length(x) ÷ (c * n)
    y = similar(x); mean = similar(x, F32, (n * G,)); rstd = similar(x, F32, (n * G,))
    check(ccall(sym(:fb_groupnorm_fwd), Int32, (PV, PV, PV, PV, PV, PV, PV, PV, Int64, Int64, Int64, Int64, Float32, Int32),
                fbctx(), fbstream(), ptr(x), ptr(γ), ptr(β), ptr(y), ptr(mean), ptr(rstd), s, c, n, G, F32(ϵ), act_code(λ)))
    return y, mean, rstd
end
function (gn::GroupNorm)(x::B200Array{F32,N}) where {N}
    _size_check(gn, x, N - 1 => gn.chs)
    first(groupnorm_fused(gn.γ, gn.β, x, gn.G, gn.ϵ, gn.λ))
end
function (l::InstanceNorm)(x::B200Array{F32,N}) where {N}
    _size_check(l, x, N - 1 => l.chs)
    c = l.chs; n = size(x, N); s = length(x) ÷ (c * n)
    if l.track_stats && _isactive(l, x) !== true
        y = similar(x)
        check(ccall(sym(:fb_batchnorm_fwd_infer), Int32, (PV, PV, PV, PV, PV, PV, PV, PV, Int64, Int64, Int64, Float32, Int32),
                    fbctx(), fbstream(), ptr(x), ptr(l.γ), ptr(l.β), ptr(l.μ), ptr(l.σ²), ptr(y), s, c, n, F32(l.ϵ), act_code(l.λ)))
        return y
    end
    y, mean, rstd = groupnorm_fused(l.γ, l.β, x, c, l.ϵ, l.λ)
    if l.track_stats
        check(ccall(sym(:fb_instancenorm_update_stats), Int32, (PV, PV, PV, PV, PV, PV, Int64, Int64, Int64, Float32, Float32),
                    fbctx(), fbstream(), ptr(mean), ptr(rstd), ptr(l.μ), ptr(l.σ²), s, c, n, F32(l.ϵ), F32(l.momentum)))
    end
    return y
end
function ChainRulesCore.rrule(::typeof(groupnorm_fused), γ, β, x::B200Array{F32,N}, G::Int, ϵ, λ) where {N}
    y, mean, rstd = groupnorm_fused(γ, β, x, G, ϵ, λ)
    c = size(x, N - 1); n = size(x, N); s = length(x) ÷ (c * n)
    function groupnorm_pullback(Δ)
        dy = unthunk(Δ[1]); dx = similar(x)
        dγ = grad_like(γ); dβ = grad_like(β)
        check(ccall(sym(:fb_groupnorm_bwd), Int32, (PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, Int64, Int64, Int64, Int64, Int32),
                    fbctx(), fbstream(), ptr(x), ptr(γ), ptr(β), ptr(mean), ptr(rstd), ptr(dy), ptr(dx), ptr(dγ), ptr(dβ), s, c, n, G, act_code(λ)))
        grad_done!(γ); grad_done!(β)
        return NoTangent(), dγ === nothing ? NoTangent() : dγ, dβ === nothing ? NoTangent() : dβ, dx, NoTangent(), NoTangent(), NoTangent()
    end
    return (y, mean, rstd), groupnorm_pullback
end
