# Losses.
# replaces mean(.-sum(y .* logsoftmax(ŷ; dims=1); dims=1))                         src/losses/functions.jl:270-273
# Returns (loss as a one-element device array, dŷ); the scalar is read back once by the caller-facing method.
function xent_fused(ŷ::B200Matrix{F32}, y::B200Matrix{F32}, want_grad::Bool)
    size(ŷ) == size(y) || throw(DimensionMismatch("loss function expects size(ŷ) = $(size(ŷ)) to match size(y) = $(size(y))"))
    c, n = size(ŷ); loss = similar(ŷ, F32, (1,)); dŷ = want_grad ? similar(ŷ) : nothing
    check(ccall(sym(:fb_logitcrossentropy_dense), Int32, (PV, PV, PV, PV, PV, PV, Int64, Int64, Float32),
                fbctx(), fbstream(), ptr(ŷ), ptr(y), ptr(loss), ptr(dŷ), c, n, 1f0))
    return loss, dŷ
end
"One-hot targets kept as 1-based Int32 labels on the device (what `onehotbatch(labels, 1:C)` stands for)."
struct OneHotLabels; labels::B200Array{Int32,1}; nclasses::Int; end
function xent_fused(ŷ::B200Matrix{F32}, y::OneHotLabels, want_grad::Bool)
    c, n = size(ŷ)
    (c == y.nclasses && n == length(y.labels)) || throw(DimensionMismatch("loss function expects size(ŷ) = $(size(ŷ)) to match size(y) = $((y.nclasses, length(y.labels)))"))
    loss = similar(ŷ, F32, (1,)); dŷ = want_grad ? similar(ŷ) : nothing
    check(ccall(sym(:fb_logitcrossentropy_labels), Int32, (PV, PV, PV, PV, PV, PV, Int64, Int64, Float32),
                fbctx(), fbstream(), ptr(ŷ), ptr(y.labels), ptr(loss), ptr(dŷ), c, n, 1f0))
    return loss, dŷ
end

function Flux.Losses.logitcrossentropy(ŷ::B200Matrix{F32}, y::Union{B200Matrix{F32},OneHotLabels}; dims=1, agg=Flux.mean)
    (dims == 1 && agg === Flux.mean) || throw(ArgumentError("logitcrossentropy on B200 arrays supports dims = 1, agg = mean"))
    return Array(first(xent_fused(ŷ, y, false)))[1]      # the one device -> host read of the step (src/train.jl:377)
end
function ChainRulesCore.rrule(::typeof(Flux.Losses.logitcrossentropy), ŷ::B200Matrix{F32}, y::Union{B200Matrix{F32},OneHotLabels}; dims=1, agg=Flux.mean)
    (dims == 1 && agg === Flux.mean) || throw(ArgumentError("logitcrossentropy on B200 arrays supports dims = 1, agg = mean"))
    loss, dŷ = xent_fused(ŷ, y, true)
    function xent_pullback(Δ)
        s = F32(unthunk(Δ))
        s == 1f0 || check(ccall(sym(:fb_scale), Int32, (PV, PV, PV, Float32, PV, Int64), fbctx(), fbstream(), ptr(dŷ), s, ptr(dŷ), length(dŷ)))
        return NoTangent(), dŷ, NoTangent()
    end
    return Array(loss)[1], xent_pullback
end
