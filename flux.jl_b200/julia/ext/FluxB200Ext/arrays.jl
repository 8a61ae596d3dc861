# The closed set of array operations that loss functions and Zygote's accumulation need on B200 arrays.  Anything
# else (broadcasts, scalar indexing) raises instead of silently running element by element on the host.

"sum(abs2, x) as a device scalar read back once (the loss of benchmark configurations 2-4)."
function Base.sum(::typeof(abs2), x::B200Array{F32})
    out = similar(x, F32, (1,))
    check(ccall(sym(:fb_sumsq), Int32, (PV, PV, PV, Int64, PV), fbctx(), fbstream(), ptr(x), length(x), ptr(out)))
    return Array(out)[1]
end
function ChainRulesCore.rrule(::typeof(sum), ::typeof(abs2), x::B200Array{F32})
    function sum_abs2_pullback(Δ)
        dx = similar(x)
        check(ccall(sym(:fb_scale), Int32, (PV, PV, PV, Float32, PV, Int64), fbctx(), fbstream(), ptr(x), 2f0 * F32(unthunk(Δ)), ptr(dx), length(x)))
        return NoTangent(), NoTangent(), dx
    end
    return sum(abs2, x), sum_abs2_pullback
end

function Base.sum(x::B200Array{F32})
    out = similar(x, F32, (1,))
    check(ccall(sym(:fb_sum), Int32, (PV, PV, PV, Int64, PV), fbctx(), fbstream(), ptr(x), length(x), ptr(out)))
    return Array(out)[1]
end
function ChainRulesCore.rrule(::typeof(sum), x::B200Array{F32})
    sum_pullback(Δ) = (NoTangent(), fill!(similar(x), F32(unthunk(Δ))))
    return sum(x), sum_pullback
end

"a + b (Zygote's `accum` of two tangents)."
function Base.:+(a::B200Array{F32,N}, b::B200Array{F32,N}) where {N}
    size(a) == size(b) || throw(DimensionMismatch("dimensions must match: a has dims $(size(a)), b has dims $(size(b))"))
    c = copy(a)
    check(ccall(sym(:fb_axpy), Int32, (PV, PV, Float32, PV, PV, Int64), fbctx(), fbstream(), 1f0, ptr(b), ptr(c), length(c)))
    return c
end
function ChainRulesCore.rrule(::typeof(+), a::B200Array{F32,N}, b::B200Array{F32,N}) where {N}
    plus_pullback(Δ) = (NoTangent(), unthunk(Δ), unthunk(Δ))
    return a + b, plus_pullback
end

"s * x and x * s for a host scalar (the cotangent `2 .* y`, learning-rate scaling)."
function Base.:*(s::Real, x::B200Array{F32})
    y = similar(x)
    check(ccall(sym(:fb_scale), Int32, (PV, PV, PV, Float32, PV, Int64), fbctx(), fbstream(), ptr(x), F32(s), ptr(y), length(x)))
    return y
end
Base.:*(x::B200Array{F32}, s::Real) = s * x
Base.:-(x::B200Array{F32}) = -1f0 * x
function ChainRulesCore.rrule(::typeof(*), s::Real, x::B200Array{F32})
    scale_pullback(Δ) = (NoTangent(), NoTangent(), s * unthunk(Δ))   # no tangent for the host scalar: it is a constant of the loss
    return s * x, scale_pullback
end

"x .-= η .* dx in one kernel (Optimisers.Descent and `subtract!`)."
function axpy!(α::Real, x::B200Array{F32}, y::B200Array{F32})
    check(ccall(sym(:fb_axpy), Int32, (PV, PV, Float32, PV, PV, Int64), fbctx(), fbstream(), F32(α), ptr(x), ptr(y), length(y)))
    return y
end

# Zygote accumulates tangents of arrays that are used twice with `accum(a, b) = a .+ b`; route that to `+`.
Base.Broadcast.broadcasted(::typeof(+), a::B200Array{F32,N}, b::B200Array{F32,N}) where {N} = a + b
Base.Broadcast.broadcasted(::typeof(*), s::Real, x::B200Array{F32}) = s * x
Base.Broadcast.broadcasted(::typeof(*), x::B200Array{F32}, s::Real) = s * x
