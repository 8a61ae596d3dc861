# Optimiser rules on B200 arrays.
# replaces the per-leaf broadcasts of Optimisers.apply!(::Adam, ...) and `x .-= dx`   src/train.jl:425
#
# Optimisers.update! calls `apply!(rule, state, x, dx)` to turn the gradient into a step and then `subtract!(x, step)`.
# The fused kernels update x in place, so apply! hands back a marker that `subtract!` treats as "already applied".
struct AppliedStep end
Optimisers.subtract!(x::B200Array, ::AppliedStep) = x
Optimisers.maywrite(::B200Array) = true
Optimisers.isnumeric(::B200Array{F32}) = true
Optimisers.init(o::Optimisers.Adam, x::B200Array{F32}) = (fill!(similar(x), 0), fill!(similar(x), 0), F32.(o.beta))

function Optimisers.apply!(o::Optimisers.Adam, (m, v, βt), x::B200Array{F32}, dx::B200Array{F32})
    ws = [x.ptr]; gs = [dx.ptr]; ms = [m.ptr]; vs = [v.ptr]; ns = Int64[length(x)]
    check(ccall(sym(:fb_adam_step), Int32, (PV, PV, Int32, Ptr{PV}, Ptr{PV}, Ptr{PV}, Ptr{PV}, Ptr{Int64}, Float32, Float32, Float32, Float32, Float32, Float32, Float32),
                fbctx(), fbstream(), Int32(1), ws, gs, ms, vs, ns, F32(o.eta), F32(o.beta[1]), F32(o.beta[2]), F32(o.epsilon), F32(βt[1]), F32(βt[2]), 1f0))
    return (m, v, βt .* F32.(o.beta)), AppliedStep()
end
function Optimisers.apply!(o::Optimisers.Descent, state, x::B200Array{F32}, dx::B200Array{F32})
    axpy!(-F32(o.eta), dx, x)
    return state, AppliedStep()
end

# `Flux.trainstep!` polls the device error word between steps: a kernel whose bounded wait ran out leaves a code
# there and its results are invalid.
function check_device_error()
    code = Ref{Int32}(0)
    check(ccall(sym(:fb_device_error), Int32, (PV, PV, Ptr{Int32}), fbctx(), fbstream(), code))
    code[] == 0 || error("a B200 kernel gave up waiting (device error code $(code[])); the results of this step are invalid")
    return nothing
end
