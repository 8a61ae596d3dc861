# B200Arrays — the trigger package of Flux's B200 extension: owns the array / device types and the handle of
# libfluxb200.so.  Loading it (next to Flux) activates ext/FluxB200Ext, exactly as `CUDA` activates FluxCUDAExt
# (Flux's Project.toml [extensions]).
#
# NOT EXECUTED in the build environment of this repository (no Julia toolchain there); every ccall signature below
# mirrors include/fluxb200.h and is exercised from Python through the same C ABI.
module B200Arrays

using Adapt, Libdl
import MLDataDevices

export B200Array, B200Device, B200Matrix, B200VecOrMat, BFloat16Bits, fbcall, fbctx, fbstream

"The raw 16-bit pattern of a BFloat16 value: the element type of arrays in BFloat16 storage (Flux.bf16)."
primitive type BFloat16Bits 16 end

const libfluxb200 = Ref{Ptr{Cvoid}}(C_NULL)
const ctx = Ref{Ptr{Cvoid}}(C_NULL)

function __init__()
    path = get(ENV, "FLUXB200_LIB", joinpath(@__DIR__, "..", "..", "..", "fluxb200", "libfluxb200.so"))
    libfluxb200[] = Libdl.dlopen(path)          # throws when the library is missing: there is no CPU fallback
end

sym(name::Symbol) = Libdl.dlsym(libfluxb200[], name)
last_error() = unsafe_string(ccall(sym(:fb_last_error), Cstring, ()))

struct FluxB200Error <: Exception
    code::Int32
    msg::String
end

check(status::Int32) = status == 0 ? nothing : throw(FluxB200Error(status, last_error()))

"Context of the current device (created on first use; one Julia process drives one GPU)."
function fbctx()
    if ctx[] == C_NULL
        out = Ref{Ptr{Cvoid}}(C_NULL)
        check(ccall(sym(:fb_ctx_create), Int32, (Int32, Ptr{Ptr{Cvoid}}), Int32(current_device[]), out))
        ctx[] = out[]
    end
    return ctx[]
end
const current_device = Ref(0)
fbstream() = C_NULL   # the default stream; a task-local stream can be returned here

# ---------------------------------------------------------------------------------------------- array type ---
mutable struct B200Array{T,N} <: AbstractArray{T,N}
    ptr::Ptr{Cvoid}
    dims::NTuple{N,Int}
    owner::Any                      # parent array for reshapes / views of the same memory
    function B200Array{T,N}(::UndefInitializer, dims::NTuple{N,Int}) where {T,N}
        out = Ref{Ptr{Cvoid}}(C_NULL)
        check(ccall(sym(:fb_malloc), Int32, (Ptr{Cvoid}, Int64, Ptr{Ptr{Cvoid}}), fbctx(), prod(dims) * sizeof(T), out))
        a = new{T,N}(out[], dims, nothing)
        finalizer(x -> ccall(sym(:fb_free), Int32, (Ptr{Cvoid}, Ptr{Cvoid}), fbctx(), x.ptr), a)
        return a
    end
    B200Array{T,N}(ptr::Ptr{Cvoid}, dims::NTuple{N,Int}, owner) where {T,N} = new{T,N}(ptr, dims, owner)
end
const B200Matrix{T} = B200Array{T,2}
const B200VecOrMat{T} = Union{B200Array{T,1},B200Array{T,2}}

Base.size(a::B200Array) = a.dims
Base.similar(a::B200Array{T}, ::Type{S}, dims::Dims{N}) where {T,S,N} = B200Array{S,N}(undef, dims)
Base.reshape(a::B200Array{T}, dims::Dims{N}) where {T,N} =
    (prod(dims) == length(a) || throw(DimensionMismatch("reshape")); B200Array{T,N}(a.ptr, dims, a))
Base.unsafe_convert(::Type{Ptr{T}}, a::B200Array{T}) where {T} = convert(Ptr{T}, a.ptr)
# scalar indexing is an error on purpose: anything that is not an explicit kernel must not silently run on the host
Base.getindex(::B200Array, I...) = error("scalar indexing of a B200Array is not supported; use Array(x)")

function B200Array(x::Array{T,N}) where {T,N}
    a = B200Array{T,N}(undef, size(x))
    check(ccall(sym(:fb_memcpy_h2d), Int32, (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int64),
                fbctx(), fbstream(), a.ptr, x, sizeof(x)))
    return a
end
function Base.Array(a::B200Array{T,N}) where {T,N}
    x = Array{T,N}(undef, size(a))
    check(ccall(sym(:fb_memcpy_d2h), Int32, (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int64),
                fbctx(), fbstream(), x, a.ptr, sizeof(x)))
    return x
end
Base.fill!(a::B200Array{Float32}, v) =
    (check(ccall(sym(:fb_fill), Int32, (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Float32, Int64), fbctx(), fbstream(), a.ptr, Float32(v), length(a))); a)
Base.zero(a::B200Array{Float32}) = fill!(similar(a), 0)
"zeros(Float32, dims...) on the device."
function zeros(::Type{T}, dims::Integer...) where {T}
    a = B200Array{T,length(dims)}(undef, Int.(dims))
    check(ccall(sym(:fb_memset), Int32, (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int32, Int64), fbctx(), fbstream(), a.ptr, Int32(0), sizeof(T) * length(a)))
    return a
end
"A view of `count = prod(dims)` elements of the flat array `a` starting at element offset `off` (0-based), shaped `dims`."
function view1d(a::B200Array{T,1}, off::Integer, dims::Dims{N}) where {T,N}
    (0 <= off && off + prod(dims) <= length(a)) || throw(BoundsError(a, off + prod(dims)))
    return B200Array{T,N}(a.ptr + off * sizeof(T), dims, a)
end
Base.copy(a::B200Array{T,N}) where {T,N} = (b = similar(a);
    check(ccall(sym(:fb_memcpy_d2d), Int32, (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int64), fbctx(), fbstream(), b.ptr, a.ptr, sizeof(T) * length(a))); b)

# --------------------------------------------------------------------------------------------- device type ---
struct B200Device <: MLDataDevices.AbstractGPUDevice end
MLDataDevices.functional(::Type{<:B200Device}) = libfluxb200[] != C_NULL
MLDataDevices.get_device(::B200Array) = B200Device()
MLDataDevices.get_device_type(::B200Array) = B200Device
MLDataDevices.set_device!(::Type{B200Device}, ::Nothing, rank::Integer) = (current_device[] = rank; nothing)   # used by FluxMPIExt.jl:17-22
Adapt.adapt_storage(::B200Device, x::Array{<:AbstractFloat}) = B200Array(Float32.(x))   # `model |> B200Device()`, like `gpu`
Adapt.adapt_storage(::B200Device, x::Array{<:Integer}) = B200Array(Int32.(x))            # index arrays (Embedding), labels
Adapt.adapt_storage(::B200Device, x::Array{Bool}) = B200Array(UInt8.(x))                 # masks
Adapt.adapt_storage(::MLDataDevices.CPUDevice, x::B200Array) = Array(x)            # `cpu(model)`

"Generic status-checked call into the library: fbcall(:fb_sumsq, (Ptr{Cvoid}, Int64, Ptr{Cvoid}), x.ptr, n, out.ptr)"
macro fbcall(name, types, args...)
    esc(:(B200Arrays.check(ccall(B200Arrays.sym($name), Int32, (Ptr{Cvoid}, Ptr{Cvoid}, $(types.args...)), B200Arrays.fbctx(), B200Arrays.fbstream(), $(args...)))))
end

end # module
