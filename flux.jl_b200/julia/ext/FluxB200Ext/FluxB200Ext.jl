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
# STATUS: written without a Julia toolchain and never executed.  What is checked mechanically (tests/test_julia_ext.py
# of the repository that ships the library) is that every `ccall` names an exported entry point of include/fluxb200.h
# with the right number of arguments and C types; the same entry points are driven from Python by the parity tests.
module FluxB200Ext

using Flux, B200Arrays, ChainRulesCore
using Flux: Chain, Dense, LayerNorm, BatchNorm, GroupNorm, InstanceNorm, Embedding, Dropout,
            LSTMCell, GRUCell, RNNCell, GRUv3Cell, _size_check, _isactive
import NNlib, Optimisers
using B200Arrays: B200Array, B200Device, B200Matrix, B200VecOrMat, check, sym, fbctx, fbstream

const F32 = Float32
const PV = Ptr{Cvoid}
ptr(a::B200Array) = a.ptr
ptr(::Union{Nothing,Bool}) = C_NULL
arr_or_nothing(b) = b isa B200Array ? b : nothing

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

# Where the pullbacks put parameter gradients: a slice of the flat gradient buffer when a GradientArena is active
# (distributed.jl), else a fresh array.  `grad_done!` tells the arena that the slice has been written.
grad_like(p::B200Array) = (a = arena[]; a !== nothing && haskey(a.view, p)) ? a.view[p] : similar(p)
grad_like(::Any) = nothing
grad_done!(p::B200Array) = (a = arena[]; a !== nothing && haskey(a.leaf_id, p) && mark_ready!(a, p); nothing)
grad_done!(::Any) = nothing

include("distributed.jl")   # defines `arena`, GradientArena, the DistributedUtils methods
include("arrays.jl")        # the closed set of array operations a loss function needs, with their rrules
include("dense.jl")
include("norms.jl")
include("recurrent.jl")
include("attention.jl")
include("loss.jl")
include("optimiser.jl")

end # module
