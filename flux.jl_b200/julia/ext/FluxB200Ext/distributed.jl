# DistributedUtils on B200 arrays.
# replaces NCCL.Allreduce! / Broadcast! / Reduce! on CuArray                       ext/FluxMPINCCLExt/FluxMPINCCLExt.jl:38-107
const DU = Flux.DistributedUtils
const comm = Ref{PV}(C_NULL)      # fb_comm*, created by `init_communicator!`

# The NCCL unique id travels over whatever host channel the launcher offers; the reference broadcasts it with MPI
# (FluxMPINCCLExt.jl:19-30).  `bcast_bytes!` must fill `id` on every rank with rank 0's bytes.
function init_communicator!(bcast_bytes!::Function, rank::Integer, nranks::Integer)
    id = zeros(UInt8, 128)
    rank == 0 && check(ccall(sym(:fb_comm_get_unique_id), Int32, (PV,), id))
    bcast_bytes!(id)
    out = Ref{PV}(C_NULL)
    check(ccall(sym(:fb_comm_init_rank), Int32, (PV, PV, Int32, Int32, Ptr{PV}), fbctx(), id, Int32(nranks), Int32(rank), out))
    comm[] = out[]
    return nothing
end

"Raises when NCCL has reported an asynchronous error on the communicator; call it between steps."
function check_async_error()
    comm[] == C_NULL && return nothing
    code = Ref{Int32}(0)
    check(ccall(sym(:fb_comm_async_error), Int32, (PV, Ptr{Int32}), comm[], code))
    code[] == 0 || error("NCCL reported asynchronous error $(code[])")
    return nothing
end

opcode(::typeof(+)) = Int32(0)
opcode(::typeof(DU.avg)) = Int32(1)
function DU.__allreduce!(::DU.NCCLBackend, buf::B200Array{F32}, op::F, ::B200Device) where {F}
    check(ccall(sym(:fb_allreduce), Int32, (PV, PV, PV, PV, Int64, Int32), comm[], fbstream(), ptr(buf), ptr(buf), length(buf), opcode(op)))
    return buf
end
function DU.__allreduce!(::DU.NCCLBackend, send::B200Array{F32}, recv::B200Array{F32}, op::F, ::B200Device) where {F}
    check(ccall(sym(:fb_allreduce), Int32, (PV, PV, PV, PV, Int64, Int32), comm[], fbstream(), ptr(send), ptr(recv), length(recv), opcode(op)))
    return recv
end
function DU.__bcast!(::DU.NCCLBackend, buf::B200Array{F32}, ::B200Device; root=0)
    check(ccall(sym(:fb_bcast), Int32, (PV, PV, PV, PV, Int64, Int32), comm[], fbstream(), ptr(buf), ptr(buf), length(buf), Int32(root)))
    return buf
end
function DU.__bcast!(::DU.NCCLBackend, send::B200Array{F32}, recv::B200Array{F32}, ::B200Device; root=0)
    check(ccall(sym(:fb_bcast), Int32, (PV, PV, PV, PV, Int64, Int32), comm[], fbstream(), ptr(send), ptr(recv), length(recv), Int32(root)))
    return recv
end
function DU.__reduce!(::DU.NCCLBackend, buf::B200Array{F32}, op::F, ::B200Device; root=0) where {F}
    check(ccall(sym(:fb_reduce), Int32, (PV, PV, PV, PV, Int64, Int32, Int32), comm[], fbstream(), ptr(buf), ptr(buf), length(buf), opcode(op), Int32(root)))
    return buf
end
function DU.__reduce!(::DU.NCCLBackend, send::B200Array{F32}, recv::B200Array{F32}, op::F, ::B200Device; root=0) where {F}
    check(ccall(sym(:fb_reduce), Int32, (PV, PV, PV, PV, Int64, Int32, Int32), comm[], fbstream(), ptr(send), ptr(recv), length(recv), opcode(op), Int32(root)))
    return recv
end

# Bucketed, overlapped gradient averaging for DistributedOptimizer                  src/distributed/public_api.jl:286-300
# Gradients of a model moved to the device live in ONE flat buffer (GradientArena); every leaf's gradient is a view
# into it, registered with the native bucket set.  The rrules write dW / db straight into those views (`grad_like`)
# and call `grad_done!`; a bucket's mean all-reduce starts on the library's communication stream as soon as its last
# leaf is ready, while the reverse sweep goes on.  `apply!` of the wrapped rule then only waits for the buckets.
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
    offs = IdDict{Any,Int}()
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
"Makes `a` the arena the pullbacks write into (call once after `Flux.setup`), or `nothing` to switch it off."
use_arena!(a) = (arena[] = a; a)
begin_step!(a::GradientArena) = check(ccall(sym(:fb_bucket_begin_step), Int32, (PV,), a.set))
mark_ready!(a::GradientArena, p) = check(ccall(sym(:fb_bucket_mark_ready), Int32, (PV, Int32, PV), a.set, a.leaf_id[p], fbstream()))
wait_all!(a::GradientArena) = check(ccall(sym(:fb_bucket_wait), Int32, (PV, PV), a.set, fbstream()))
destroy!(a::GradientArena) = (check(ccall(sym(:fb_bucket_destroy), Int32, (PV,), a.set)); arena[] === a && (arena[] = nothing); nothing)

function Optimisers.apply!(o::DU.DistributedOptimizer{<:DU.NCCLBackend}, state, x::B200Array{F32}, dx::B200Array{F32})
    a = arena[]
    if a !== nothing && haskey(a.view, x) && ptr(a.view[x]) == ptr(dx)
        wait_all!(a)                                       # averaged in its bucket already: do not reduce twice
    else
        DU.allreduce!(o.backend, dx, DU.avg)
    end
    return Optimisers.apply!(o.opt, state, x, dx)
end
