# Recurrence: scan over LSTMCell / GRUCell / RNNCell / GRUv3Cell.
# replaces scan(cell, x, state): the host loop over eachslice(x, dims=2)          src/layers/recurrent.jl:1-8
cache_floats(f::Symbol, in, H, T, B) = max(ccall(sym(f), Int64, (Int64, Int64, Int64, Int64), in, H, T, B) ÷ 4, 1)
state_or_null(h, H, B) = (h isa B200Array && size(h) == (H, B)) ? h : nothing   # a zero vector state (initialstates) means NULL = zeros

function lstm_scan(cell::LSTMCell, x::B200Array{F32,3}, h0, c0, cache)
    in, T, B = size(x); H = size(cell.Wh, 2)
    out = similar(x, F32, (H, T, B)); hT = similar(x, F32, (H, B)); cT = similar(hT)
    check(ccall(sym(:fb_lstm_fwd), Int32, (PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, Int64, Int64, Int64, Int64),
                fbctx(), fbstream(), ptr(cell.Wi), ptr(cell.Wh), ptr(arr_or_nothing(cell.bias)), ptr(x), ptr(h0), ptr(c0), ptr(out), ptr(hT), ptr(cT),
                ptr(cache), in, H, T, B))
    return out, hT, cT
end
function Flux.scan(cell::LSTMCell{<:B200Matrix}, x::B200Array{F32,3}, (h, c))
    H = size(cell.Wh, 2); B = size(x, 3)
    out, hT, cT = lstm_scan(cell, x, state_or_null(h, H, B), state_or_null(c, H, B), nothing)
    return out, (hT, cT)
end
function ChainRulesCore.rrule(::typeof(lstm_scan), cell::LSTMCell, x::B200Array{F32,3}, h0, c0, _)
    in, T, B = size(x); H = size(cell.Wh, 2)
    cache = similar(x, F32, (cache_floats(:fb_lstm_cache_bytes, in, H, T, B),))
    out, hT, cT = lstm_scan(cell, x, h0, c0, cache)
    b = arr_or_nothing(cell.bias)
    function lstm_pullback(Δ)
        dout, dhT, dcT = map(t -> t isa AbstractZero ? nothing : unthunk(t), (Δ[1], Δ[2], Δ[3]))
        dout === nothing && (dout = fill!(similar(out), 0))
        dWi = grad_like(cell.Wi); dWh = grad_like(cell.Wh); db = b === nothing ? nothing : grad_like(b); dx = similar(x)
        check(ccall(sym(:fb_lstm_bwd), Int32, (PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, Int64, Int64, Int64, Int64),
                    fbctx(), fbstream(), ptr(cell.Wi), ptr(cell.Wh), ptr(x), ptr(h0), ptr(c0), ptr(out), ptr(cache), ptr(dout), ptr(dhT), ptr(dcT),
                    ptr(dWi), ptr(dWh), ptr(db), ptr(dx), in, H, T, B))
        grad_done!(cell.Wi); grad_done!(cell.Wh); grad_done!(b)
        dcell = Tangent{typeof(cell)}(; Wi=dWi, Wh=dWh, bias=db === nothing ? NoTangent() : db)
        return NoTangent(), dcell, dx, NoTangent(), NoTangent(), NoTangent()
    end
    return (out, hT, cT), lstm_pullback
end

function gru_scan(cell::GRUCell, x::B200Array{F32,3}, h0, cache)
    in, T, B = size(x); H = size(cell.Wh, 2)
    out = similar(x, F32, (H, T, B)); hT = similar(x, F32, (H, B))
    check(ccall(sym(:fb_gru_fwd), Int32, (PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, Int64, Int64, Int64, Int64),
                fbctx(), fbstream(), ptr(cell.Wi), ptr(cell.Wh), ptr(arr_or_nothing(cell.b)), ptr(x), ptr(h0), ptr(out), ptr(hT), ptr(cache), in, H, T, B))
    return out, hT
end
function Flux.scan(cell::GRUCell{<:B200Matrix}, x::B200Array{F32,3}, h)
    out, hT = gru_scan(cell, x, state_or_null(h, size(cell.Wh, 2), size(x, 3)), nothing)
    return out, hT
end
function ChainRulesCore.rrule(::typeof(gru_scan), cell::GRUCell, x::B200Array{F32,3}, h0, _)
    in, T, B = size(x); H = size(cell.Wh, 2)
    cache = similar(x, F32, (cache_floats(:fb_gru_cache_bytes, in, H, T, B),))
    out, hT = gru_scan(cell, x, h0, cache)
    b = arr_or_nothing(cell.b)
    function gru_pullback(Δ)
        dout, dhT = map(t -> t isa AbstractZero ? nothing : unthunk(t), (Δ[1], Δ[2]))
        dout === nothing && (dout = fill!(similar(out), 0))
        dWi = grad_like(cell.Wi); dWh = grad_like(cell.Wh); db = b === nothing ? nothing : grad_like(b); dx = similar(x)
        check(ccall(sym(:fb_gru_bwd), Int32, (PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, Int64, Int64, Int64, Int64),
                    fbctx(), fbstream(), ptr(cell.Wi), ptr(cell.Wh), ptr(x), ptr(h0), ptr(out), ptr(cache), ptr(dout), ptr(dhT), ptr(dWi), ptr(dWh),
                    ptr(db), ptr(dx), in, H, T, B))
        grad_done!(cell.Wi); grad_done!(cell.Wh); grad_done!(b)
        dcell = Tangent{typeof(cell)}(; Wi=dWi, Wh=dWh, b=db === nothing ? NoTangent() : db)
        return NoTangent(), dcell, dx, NoTangent(), NoTangent()
    end
    return (out, hT), gru_pullback
end

# RNNCell (recurrent.jl:193-198)
function rnn_scan(cell::RNNCell, x::B200Array{F32,3}, h0)
    in, T, B = size(x); H = size(cell.Wh, 2)
    out = similar(x, F32, (H, T, B)); hT = similar(x, F32, (H, B))
    check(ccall(sym(:fb_rnn_fwd), Int32, (PV, PV, Int32, PV, PV, PV, PV, PV, PV, PV, Int64, Int64, Int64, Int64),
                fbctx(), fbstream(), act_code(cell.σ), ptr(cell.Wi), ptr(cell.Wh), ptr(arr_or_nothing(cell.bias)), ptr(x), ptr(h0), ptr(out), ptr(hT), in, H, T, B))
    return out, hT
end
Flux.scan(cell::RNNCell{<:Any,<:B200Matrix}, x::B200Array{F32,3}, h) = rnn_scan(cell, x, state_or_null(h, size(cell.Wh, 2), size(x, 3)))
function ChainRulesCore.rrule(::typeof(rnn_scan), cell::RNNCell, x::B200Array{F32,3}, h0)
    in, T, B = size(x); H = size(cell.Wh, 2)
    out, hT = rnn_scan(cell, x, h0)
    b = arr_or_nothing(cell.bias)
    function rnn_pullback(Δ)
        dout, dhT = map(t -> t isa AbstractZero ? nothing : unthunk(t), (Δ[1], Δ[2]))
        dout === nothing && (dout = fill!(similar(out), 0))
        scratch = similar(x, F32, (cache_floats(:fb_rnn_cache_bytes, in, H, T, B),))
        dWi = grad_like(cell.Wi); dWh = grad_like(cell.Wh); db = b === nothing ? nothing : grad_like(b); dx = similar(x)
        check(ccall(sym(:fb_rnn_bwd), Int32, (PV, PV, Int32, PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, Int64, Int64, Int64, Int64),
                    fbctx(), fbstream(), act_code(cell.σ), ptr(cell.Wi), ptr(cell.Wh), ptr(x), ptr(h0), ptr(out), ptr(scratch), ptr(dout), ptr(dhT),
                    ptr(dWi), ptr(dWh), ptr(db), ptr(dx), in, H, T, B))
        grad_done!(cell.Wi); grad_done!(cell.Wh); grad_done!(b)
        dcell = Tangent{typeof(cell)}(; Wi=dWi, Wh=dWh, bias=db === nothing ? NoTangent() : db)
        return NoTangent(), dcell, dx, NoTangent()
    end
    return (out, hT), rnn_pullback
end

# GRUv3Cell (recurrent.jl:795-809)
function gruv3_scan(cell::GRUv3Cell, x::B200Array{F32,3}, h0, cache)
    in, T, B = size(x); H = size(cell.Wh, 2)
    out = similar(x, F32, (H, T, B)); hT = similar(x, F32, (H, B))
    check(ccall(sym(:fb_gruv3_fwd), Int32, (PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, Int64, Int64, Int64, Int64),
                fbctx(), fbstream(), ptr(cell.Wi), ptr(cell.Wh), ptr(arr_or_nothing(cell.b)), ptr(cell.Wh_h̃), ptr(x), ptr(h0), ptr(out), ptr(hT), ptr(cache),
                in, H, T, B))
    return out, hT
end
Flux.scan(cell::GRUv3Cell{<:B200Matrix}, x::B200Array{F32,3}, h) = gruv3_scan(cell, x, state_or_null(h, size(cell.Wh, 2), size(x, 3)), nothing)
function ChainRulesCore.rrule(::typeof(gruv3_scan), cell::GRUv3Cell, x::B200Array{F32,3}, h0, _)
    in, T, B = size(x); H = size(cell.Wh, 2)
    cache = similar(x, F32, (cache_floats(:fb_gruv3_cache_bytes, in, H, T, B),))
    out, hT = gruv3_scan(cell, x, h0, cache)
    b = arr_or_nothing(cell.b)
    function gruv3_pullback(Δ)
        dout, dhT = map(t -> t isa AbstractZero ? nothing : unthunk(t), (Δ[1], Δ[2]))
        dout === nothing && (dout = fill!(similar(out), 0))
        dWi = grad_like(cell.Wi); dWh = grad_like(cell.Wh); dWhh = grad_like(cell.Wh_h̃); db = b === nothing ? nothing : grad_like(b); dx = similar(x)
        check(ccall(sym(:fb_gruv3_bwd), Int32, (PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, PV, Int64, Int64, Int64, Int64),
                    fbctx(), fbstream(), ptr(cell.Wi), ptr(cell.Wh), ptr(cell.Wh_h̃), ptr(x), ptr(h0), ptr(out), ptr(cache), ptr(dout), ptr(dhT),
                    ptr(dWi), ptr(dWh), ptr(db), ptr(dWhh), ptr(dx), in, H, T, B))
        grad_done!(cell.Wi); grad_done!(cell.Wh); grad_done!(cell.Wh_h̃); grad_done!(b)
        dcell = Tangent{typeof(cell)}(; Wi=dWi, Wh=dWh, b=db === nothing ? NoTangent() : db, Wh_h̃=dWhh)
        return NoTangent(), dcell, dx, NoTangent(), NoTangent()
    end
    return (out, hT), gruv3_pullback
end
