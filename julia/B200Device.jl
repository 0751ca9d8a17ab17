# B200Device.jl -- the Julia side of libluminal_b200.so.
#
# Luminal.jl has no FFI; a backend enters through multiple dispatch on the device type
# (src/Device.jl:9-16, 82-121) and on the array type inside execute_op! (src/Execution.jl:274-371,
# 521, 566, 604).  This file is that entry: include it after "Device.jl" in src/Luminal.jl.  It adds
#   * B200Device <: AbstractDevice and B200Array (what CuArray is to CUDADevice),
#   * to_device / from_device for them,
#   * one execute_op! method per op type, each a single ccall,
#   * compile_b200 / decode helpers over the session API for the generation loop.
# Graph, NN.jl, Whisper.jl and Decoding.jl stay as they are.
#
# Every ccall below names one entry point of include/luminal_b200.h with the argument types of its
# declaration; luminal.jl_b200/_lib.py binds the same entry points with ctypes and is what the test
# suite runs (there is no Julia where this library is built).
module B200

using ..Luminal
using ..Luminal: AbstractDevice, Graph, realized_dims

const LIB = get(ENV, "LUMINAL_B200_LIB", "libluminal_b200.so")

# ---------------------------------------------------------------------------------------------
# errors: every entry point returns a status; the message is thread-local in the library
# ---------------------------------------------------------------------------------------------
struct B200Error <: Exception
    code::Int32
    msg::String
end
Base.showerror(io::IO, e::B200Error) = print(io, "libluminal_b200 error ", e.code, ": ", e.msg)
check(rc::Int32) = rc == 0 ? nothing :
    throw(B200Error(rc, unsafe_string(ccall((:lmb200_last_error, LIB), Cstring, ()))))

const F32, BF16 = Int32(0), Int32(1)
const ROWMAJOR, COLMAJOR = Int32(0), Int32(1)      # Julia arrays are column-major: always pass COLMAJOR

# ---------------------------------------------------------------------------------------------
# device and arrays
# ---------------------------------------------------------------------------------------------
struct B200Device <: AbstractDevice                # next to CPUDevice / CUDADevice (src/Device.jl:12-16)
    ctx::UInt64
end
function B200Device(ordinal::Integer=0)
    h = Ref{UInt64}(0)
    check(ccall((:lmb200_init, LIB), Int32, (Int32, Ref{UInt64}), ordinal, h))
    B200Device(h[])
end
shutdown(d::B200Device) = check(ccall((:lmb200_shutdown, LIB), Int32, (UInt64,), d.ctx))
sync(d::B200Device) = check(ccall((:lmb200_sync, LIB), Int32, (UInt64,), d.ctx))
function device_count()
    n = Ref{Int32}(0)
    check(ccall((:lmb200_device_count, LIB), Int32, (Ref{Int32},), n))
    Int(n[])
end

mutable struct B200Array{N}
    dev::B200Device
    ptr::Ptr{Cvoid}
    dims::NTuple{N,Int}
end
Base.size(a::B200Array) = a.dims
Base.ndims(::B200Array{N}) where {N} = N
dims64(a::B200Array) = collect(Int64, a.dims)
dims64(t::Tuple) = collect(Int64, t)

function alloc(d::B200Device, dims::NTuple{N,Int}) where {N}
    p = Ref{Ptr{Cvoid}}(C_NULL)
    check(ccall((:lmb200_alloc, LIB), Int32, (UInt64, Int64, Ref{Ptr{Cvoid}}), d.ctx, 4 * prod(dims), p))
    a = B200Array{N}(d, p[], dims)
    finalizer(x -> ccall((:lmb200_free, LIB), Int32, (UInt64, Ptr{Cvoid}), x.dev.ctx, x.ptr), a)
    a
end

# to_device / from_device (src/Device.jl:82-105).  The library keeps row-major tensors over the
# LOGICAL shape and re-lays the column-major image out on the way in and out.
function Luminal.to_device(a::Array{Float32,N}, d::B200Device) where {N}
    out = alloc(d, size(a))
    check(ccall((:lmb200_upload, LIB), Int32,
                (UInt64, Ptr{Cvoid}, Int32, Ptr{Float32}, Int32, Ptr{Int64}, Int32),
                d.ctx, out.ptr, F32, a, N, dims64(size(a)), COLMAJOR))
    out
end
Luminal.to_device(a::AbstractArray, d::B200Device) = Luminal.to_device(convert(Array{Float32}, a), d)
Luminal.to_device(a::B200Array, ::B200Device) = a
Luminal.to_device(x::Dict, d::B200Device) = Dict(k => Luminal.to_device(v, d) for (k, v) in x)
function Luminal.from_device(a::B200Array{N}) where {N}
    out = Array{Float32}(undef, a.dims...)
    check(ccall((:lmb200_download, LIB), Int32,
                (UInt64, Ptr{Float32}, Ptr{Cvoid}, Int32, Int32, Ptr{Int64}, Int32),
                a.dev.ctx, out, a.ptr, F32, N, dims64(a), COLMAJOR))
    out
end

# execute_with_capture (src/Device.jl:106-121; CompiledGraph hands it its steps and its cache, src/Compiler.jl:91-98):
# the first call runs f() as it is and then records it into a CUDA graph, every later call is one replay of
# cache[:cuda_exec].  If f() makes a call that cannot be recorded, cache[:cuda_exec] is `nothing` and f() keeps running
# call by call.
function Luminal.execute_with_capture(d::B200Device, f, cache::Dict)
    g = get(cache, :cuda_exec, nothing)
    if g !== nothing
        check(ccall((:lmb200_graph_launch, LIB), Int32, (UInt64, UInt64), d.ctx, g))
        return
    end
    f()
    haskey(cache, :cuda_exec) && return
    check(ccall((:lmb200_capture_begin, LIB), Int32, (UInt64,), d.ctx))
    h = Ref{UInt64}(0)
    recorded = try f(); true catch; false end
    rc = ccall((:lmb200_capture_end, LIB), Int32, (UInt64, Ref{UInt64}), d.ctx, h)
    cache[:cuda_exec] = (recorded && rc == 0) ? h[] : nothing
    if !recorded && rc == 0
        check(ccall((:lmb200_graph_destroy, LIB), Int32, (UInt64, UInt64), d.ctx, h[]))
    end
end

# ---------------------------------------------------------------------------------------------
# execute_op!: one method per op type (src/Execution.jl:274-371, 481-618), selected by the array type
# ---------------------------------------------------------------------------------------------
const NUL = Ptr{Cvoid}(C_NULL)
function ew!(out::B200Array, opcode::Integer, a::B200Array, b=nothing, c=nothing)
    e = Int64[]
    check(ccall((:lmb200_ew, LIB), Int32,
                (UInt64, Int32, Ptr{Cvoid}, Int32, Ptr{Int64}, Ptr{Cvoid}, Int32, Ptr{Int64},
                 Ptr{Cvoid}, Int32, Ptr{Int64}, Ptr{Cvoid}, Int32, Ptr{Int64}),
                out.dev.ctx, opcode, out.ptr, ndims(out), dims64(out), a.ptr, ndims(a), dims64(a),
                b === nothing ? NUL : b.ptr, b === nothing ? 0 : ndims(b), b === nothing ? e : dims64(b),
                c === nothing ? NUL : c.ptr, c === nothing ? 0 : ndims(c), c === nothing ? e : dims64(c)))
    out
end
# opcodes: the LMB200_OP_* enum of the header
Luminal.execute_op!(out::B200Array, ::Luminal.Add, a, b)            = ew!(out, 0, a, b)
Luminal.execute_op!(out::B200Array, ::Luminal.Mul, a, b)            = ew!(out, 1, a, b)
Luminal.execute_op!(out::B200Array, ::Luminal.Mod, a, b)            = ew!(out, 2, a, b)
Luminal.execute_op!(out::B200Array, ::Luminal.LessThan, a, b)       = ew!(out, 3, a, b)
Luminal.execute_op!(out::B200Array, ::Luminal.Max, a, b)            = ew!(out, 4, a, b)
Luminal.execute_op!(out::B200Array, ::Luminal.Log2, a)              = ew!(out, 8, a)
Luminal.execute_op!(out::B200Array, ::Luminal.Exp2, a)              = ew!(out, 9, a)
Luminal.execute_op!(out::B200Array, ::Luminal.Sin, a)               = ew!(out, 10, a)
Luminal.execute_op!(out::B200Array, ::Luminal.Cos, a)               = ew!(out, 11, a)
Luminal.execute_op!(out::B200Array, ::Luminal.Sqrt, a)              = ew!(out, 12, a)
Luminal.execute_op!(out::B200Array, ::Luminal.Recip, a)             = ew!(out, 13, a)
Luminal.execute_op!(out::B200Array, ::Luminal.ReLU, a)              = ew!(out, 14, a)
Luminal.execute_op!(out::B200Array, ::Luminal.Contiguous, a)        = ew!(out, 15, a)
Luminal.execute_op!(out::B200Array, ::Luminal.FusedMulAdd, a, b, c) = ew!(out, 16, a, b, c)
Luminal.execute_op!(out::B200Array, ::Luminal.FusedAddReLU, a, b)   = ew!(out, 17, a, b)

function reduce!(out::B200Array, kind::Integer, dim::Integer, a::B200Array)
    check(ccall((:lmb200_reduce, LIB), Int32, (UInt64, Int32, Ptr{Cvoid}, Ptr{Cvoid}, Int32, Ptr{Int64}, Int32),
                out.dev.ctx, kind, out.ptr, a.ptr, ndims(a), dims64(a), dim - 1))
    out
end
Luminal.execute_op!(out::B200Array, op::Luminal.SumReduce, a) = reduce!(out, 0, op.dim, a)
Luminal.execute_op!(out::B200Array, op::Luminal.MaxReduce, a) = reduce!(out, 1, op.dim, a)

function Luminal.execute_op!(out::B200Array, ::Luminal.MatMul, a::B200Array, b::B200Array)     # batch_matmul, :12-90
    check(ccall((:lmb200_matmul, LIB), Int32,
                (UInt64, Ptr{Cvoid}, Ptr{Cvoid}, Int32, Ptr{Int64}, Ptr{Cvoid}, Int32, Ptr{Int64}),
                out.dev.ctx, out.ptr, a.ptr, ndims(a), dims64(a), b.ptr, ndims(b), dims64(b)))
    out
end
function Luminal.execute_op!(out::B200Array, op::Luminal.Permute, a::B200Array)
    check(ccall((:lmb200_permute, LIB), Int32, (UInt64, Ptr{Cvoid}, Ptr{Cvoid}, Int32, Ptr{Int64}, Ptr{Int32}),
                out.dev.ctx, out.ptr, a.ptr, ndims(a), dims64(a), collect(Int32, op.dims) .- Int32(1)))
    out
end
function Luminal.execute_op!(out::B200Array, op::Luminal.Reshape, a::B200Array)              # column-major order kept, :228
    check(ccall((:lmb200_reshape_colmajor, LIB), Int32,
                (UInt64, Ptr{Cvoid}, Ptr{Cvoid}, Int32, Ptr{Int64}, Int32, Ptr{Int64}),
                out.dev.ctx, out.ptr, a.ptr, ndims(a), dims64(a), ndims(out), dims64(out)))
    out
end
function Luminal.execute_op!(out::B200Array, op::Luminal.Expand, a::B200Array)
    check(ccall((:lmb200_expand, LIB), Int32, (UInt64, Ptr{Cvoid}, Ptr{Cvoid}, Int32, Ptr{Int64}, Int32, Int64),
                out.dev.ctx, out.ptr, a.ptr, ndims(a), dims64(a), op.dim - 1, op.size))
    out
end
function Luminal.execute_op!(out::B200Array, op::Luminal.Slice, a::B200Array)                # ranges are 0-based [start, stop)
    starts = Int64[r[1] for r in op.ranges]
    stops = Int64[min(r[2], d) for (r, d) in zip(op.ranges, a.dims)]
    check(ccall((:lmb200_slice, LIB), Int32, (UInt64, Ptr{Cvoid}, Ptr{Cvoid}, Int32, Ptr{Int64}, Ptr{Int64}, Ptr{Int64}),
                out.dev.ctx, out.ptr, a.ptr, ndims(a), dims64(a), starts, stops))
    out
end
function Luminal.execute_op!(out::B200Array, op::Luminal.Pad, a::B200Array)
    check(ccall((:lmb200_pad, LIB), Int32, (UInt64, Ptr{Cvoid}, Ptr{Cvoid}, Int32, Ptr{Int64}, Ptr{Int64}, Ptr{Int64}),
                out.dev.ctx, out.ptr, a.ptr, ndims(a), dims64(a), Int64[p[1] for p in op.padding], Int64[p[2] for p in op.padding]))
    out
end
function Luminal.execute_op!(out::B200Array, op::Luminal.Unfold, a::B200Array)               # 1-D, :481-550
    check(ccall((:lmb200_unfold1d, LIB), Int32, (UInt64, Ptr{Cvoid}, Ptr{Cvoid}, Int64, Int64, Int64, Int64, Int64),
                out.dev.ctx, out.ptr, a.ptr, prod(a.dims[1:end-1]), a.dims[end],
                op.kernel_shape[1], op.stride_shape[1], op.dilation_shape[1]))
    out
end
function Luminal.execute_op!(out::B200Array, op::Luminal.FlashAttentionOp, q::B200Array, k::B200Array, v::B200Array)
    B, H, S, D = q.dims                                                                     # :374-479, 565-578
    check(ccall((:lmb200_flash_attention, LIB), Int32,
                (UInt64, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int32, Int64, Int64, Int64, Int64, Float32, Int32),
                out.dev.ctx, out.ptr, q.ptr, k.ptr, v.ptr, F32, B, H, S, D, Float32(op.scale), op.causal ? 1 : 0))
    out
end
function Luminal.execute_op!(out::B200Array, op::Luminal.Function, args::B200Array...)
    if op.name == "Gather"                                                                  # :262-264, 580-611
        table, ids = args
        check(ccall((:lmb200_gather, LIB), Int32, (UInt64, Ptr{Cvoid}, Ptr{Cvoid}, Int64, Int64, Ptr{Cvoid}, Int64),
                    out.dev.ctx, out.ptr, table.ptr, table.dims[1], table.dims[2], ids.ptr, prod(ids.dims)))
    elseif op.name == "CumSum"                                                              # :265-266, 612-613
        a = args[1]
        check(ccall((:lmb200_cumsum_last, LIB), Int32, (UInt64, Ptr{Cvoid}, Ptr{Cvoid}, Int64, Int64),
                    out.dev.ctx, out.ptr, a.ptr, prod(a.dims) ÷ a.dims[end], a.dims[end]))
    else
        error("Function op with name $(op.name) not implemented.")
    end
    out
end

# compile()'s fusion groups (src/Compiler.jl:196-215, 323-357): the group's postfix program goes to one
# kernel.  ops / args as the header lists them; inputs are the group's leaves.
function fused_ew!(out::B200Array, ops::Vector{Int32}, args::Vector{Float32}, inputs::Vector{<:B200Array})
    ptrs = Ptr{Cvoid}[a.ptr for a in inputs]
    ranks = Int32[ndims(a) for a in inputs]
    dims = Int64[d for a in inputs for d in a.dims]
    check(ccall((:lmb200_fused_ew, LIB), Int32,
                (UInt64, Ptr{Cvoid}, Int32, Ptr{Int64}, Int32, Ptr{Ptr{Cvoid}}, Ptr{Int32}, Ptr{Int64}, Int32, Ptr{Int32}, Ptr{Float32}),
                out.dev.ctx, out.ptr, ndims(out), dims64(out), length(inputs), ptrs, ranks, dims, length(ops), ops, args))
    out
end
# the norm and gate patterns compile() recognises (src/NN.jl:138-173, 246-249)
function rmsnorm_scale!(y::B200Array, x::B200Array, w::B200Array, eps::Real)
    check(ccall((:lmb200_rmsnorm_scale, LIB), Int32, (UInt64, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int64, Int64, Float32),
                y.dev.ctx, y.ptr, x.ptr, w.ptr, prod(x.dims[1:end-1]), x.dims[end], Float32(eps)))
    y
end
function layernorm!(y::B200Array, x::B200Array, w::B200Array, b::Union{B200Array,Nothing}, eps::Real)
    check(ccall((:lmb200_layernorm, LIB), Int32, (UInt64, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int64, Int64, Float32),
                y.dev.ctx, y.ptr, x.ptr, w.ptr, b === nothing ? NUL : b.ptr, prod(x.dims[1:end-1]), x.dims[end], Float32(eps)))
    y
end
function silu_gate!(out::B200Array, gate::B200Array, up::B200Array)
    check(ccall((:lmb200_silu_gate, LIB), Int32, (UInt64, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int64),
                out.dev.ctx, out.ptr, gate.ptr, up.ptr, prod(out.dims)))
    out
end

# ---------------------------------------------------------------------------------------------
# the session API: what the generation loop calls instead of building a graph per token
# (examples/llama.jl:39-99, src/Decoding.jl:91-130)
# ---------------------------------------------------------------------------------------------
struct ModelConfig                                  # lmb200_model_config, field for field
    n_layers::Int32; hidden::Int32; n_heads::Int32; n_kv_heads::Int32; head_dim::Int32
    intermediate::Int32; vocab::Int32; rms_eps::Float32; rope_base::Float32
    dtype::Int32; tp_size::Int32; tp_rank::Int32; arch::Int32; max_positions::Int32; cross_len::Int32
    reserved::Int32
end

mutable struct Model
    h::UInt64
end
function Model(d::B200Device, cfg::ModelConfig)
    h = Ref{UInt64}(0)
    check(ccall((:lmb200_model_create, LIB), Int32, (UInt64, Ref{ModelConfig}, Ref{UInt64}), d.ctx, Ref(cfg), h))
    Model(h[])
end
# full logical tensors in Julia memory order, under the registry names of src/NN.jl:180-225
function set_weight!(m::Model, name::AbstractString, w::Array{Float32})
    check(ccall((:lmb200_model_set_weight, LIB), Int32, (UInt64, Cstring, Ptr{Float32}, Int32, Ptr{Int64}, Int32),
                m.h, name, w, ndims(w), dims64(size(w)), COLMAJOR))
end
function missing_weights(m::Model)
    buf = Vector{UInt8}(undef, 1 << 20); n = Ref{Int32}(0)
    check(ccall((:lmb200_model_missing_weights, LIB), Int32, (UInt64, Ptr{UInt8}, Int64, Ref{Int32}), m.h, buf, length(buf), n))
    filter(!isempty, split(unsafe_string(pointer(buf)), '\n'))
end
init_random!(m::Model, seed::Integer, sigma::Real) =
    check(ccall((:lmb200_model_init_random, LIB), Int32, (UInt64, UInt64, Float32), m.h, seed, sigma))
destroy(m::Model) = check(ccall((:lmb200_model_destroy, LIB), Int32, (UInt64,), m.h))

mutable struct Session
    h::UInt64
    batch::Int
    vocab::Int
end
function Session(m::Model, cfg::ModelConfig, batch::Integer, max_ctx::Integer)
    h = Ref{UInt64}(0)
    check(ccall((:lmb200_session_create, LIB), Int32, (UInt64, Int32, Int32, Ref{UInt64}), m.h, batch, max_ctx, h))
    Session(h[], batch, cfg.vocab)
end
destroy(s::Session) = check(ccall((:lmb200_session_destroy, LIB), Int32, (UInt64,), s.h))
reset!(s::Session) = check(ccall((:lmb200_session_reset, LIB), Int32, (UInt64,), s.h))
set_position!(s::Session, pos::Integer) = check(ccall((:lmb200_session_set_position, LIB), Int32, (UInt64, Int32), s.h, pos))

# tokens: (batch, n) matrix of 0-based ids (the reference carries them as Float32, src/Execution.jl:263)
function prefill!(s::Session, tokens::AbstractMatrix)
    t = permutedims(Int32.(tokens))                # [batch, n] row-major = (n, batch) in Julia memory
    logits = Matrix{Float32}(undef, s.vocab, s.batch)
    check(ccall((:lmb200_prefill, LIB), Int32, (UInt64, Ptr{Int32}, Int32, Ptr{Float32}), s.h, t, size(tokens, 2), logits))
    permutedims(logits)                            # (batch, vocab)
end
function decode_step!(s::Session, tokens::Vector{Int32})
    nxt = similar(tokens)
    check(ccall((:lmb200_decode_step, LIB), Int32, (UInt64, Ptr{Int32}, Ptr{Int32}, Ptr{Float32}), s.h, tokens, nxt, C_NULL))
    nxt
end
function decode_n!(s::Session, first::Vector{Int32}, n_steps::Integer)
    out = Matrix{Int32}(undef, s.batch, n_steps)   # [n_steps, batch] row-major
    check(ccall((:lmb200_decode_n, LIB), Int32, (UInt64, Ptr{Int32}, Int32, Ptr{Int32}), s.h, first, n_steps, out))
    out
end
# greedy_decode's loop with its two exits (src/Decoding.jl:93-95, 126-129)
function decode_until!(s::Session, first::Vector{Int32}, max_steps::Integer, eot::Integer)
    out = Matrix{Int32}(undef, s.batch, max_steps); done = Ref{Int32}(0)
    check(ccall((:lmb200_decode_until, LIB), Int32, (UInt64, Ptr{Int32}, Int32, Int32, Ptr{Int32}, Ref{Int32}),
                s.h, first, max_steps, eot, out, done))
    out[:, 1:done[]]
end
# greedy_decode's loop (src/Decoding.jl:85-130) on a Whisper session created with max_ctx = MAX_TARGET_POSITION - 1 whose
# cross K/V are set: as in the reference only the LAST id of the start sequence is fed, at position length(tokens) - 1,
# over a cache whose earlier slots are still the zero rows of a fresh KVCacheState (a fresh session's cache is zeroed);
# the loop ends with the step that produced eot_id, after max_len steps, or at the position cap.  Returns the ids, the
# start sequence included; the tokenizer calls around the loop stay in Decoding.jl.
function greedy_decode!(s::Session, tokens::Vector{Int}, eot_id::Integer; max_len::Integer=448, max_positions::Integer=448)
    pos = length(tokens) - 1
    steps = min(max_len, (max_positions - 1) - pos)
    steps <= 0 && return tokens
    set_position!(s, pos)
    out = decode_until!(s, fill(Int32(tokens[end]), s.batch), steps, eot_id)
    for t in out[1, :]
        push!(tokens, Int(t))
        t == eot_id && break
    end
    tokens
end
# Whisper: cross K/V of one layer, (B, H, T, D) Julia arrays as project_cross_kv returns them (src/Whisper.jl:809-831)
function set_cross_kv!(s::Session, layer::Integer, k::Array{Float32,4}, v::Array{Float32,4})
    check(ccall((:lmb200_session_set_cross_kv, LIB), Int32, (UInt64, Int32, Ptr{Float32}, Ptr{Float32}, Int32),
                s.h, layer, k, v, COLMAJOR))
end

# compile_b200: from a model object and its WeightRegistry (src/NN.jl:180-225) to a fused session.
# `weights` maps registry names to Float32 arrays (what load_weights! puts into graph.tensors).
function compile_b200(d::B200Device, cfg::ModelConfig, weights::Dict{String,<:Array{Float32}}, batch::Integer, max_ctx::Integer)
    m = Model(d, cfg)
    for (name, w) in weights
        try
            set_weight!(m, name, w)
        catch e
            (e isa B200Error && e.code == -7) || rethrow()      # LMB200_ENOTFOUND: not a tensor of this model
        end
    end
    miss = missing_weights(m)
    isempty(miss) || @warn "Missing weights" missing_keys = miss   # as load_weights! does (src/Weights.jl:86-91)
    m, Session(m, cfg, batch, max_ctx)
end

# compile_b200 from the graph alone: Graph.nodes flattened into lmb200_node_list, recognised by the library's
# structural matchers (lmb200_match_decoder for NN.Llama / NN.Phi3, lmb200_match_whisper_step for the graph of
# build_decode_step!, src/Whisper.jl:687-742) and turned into a model + session (lmb200_compile_node_list).  The
# weights are whatever load_weights! put into graph.tensors (src/Weights.jl:60-114); for a Whisper step graph the
# encoder K/V inputs that have data there are uploaded too, and max_ctx = 0 takes the graph's max_seq.  A graph the matcher does not
# recognise raises B200Error with code -8 (LMB200_ENOMATCH): run it with compile() / execute() instead.
struct NodeList                                     # lmb200_node_list, field for field
    n_nodes::Int32; reserved::Int32
    op::Ptr{Int32}; in_off::Ptr{Int32}; in_node::Ptr{Int32}; shape_off::Ptr{Int32}; shape::Ptr{Int64}
    arg_off::Ptr{Int32}; arg::Ptr{Float64}
end
struct DecoderMatch                                 # lmb200_decoder_match
    arch::Int32; batch::Int32; seq::Int32; prev_seq::Int32; tokens_node::Int32; n_weights::Int32; max_seq::Int32; cross_len::Int32
end
const NODE_CODES = Dict{DataType,Int32}(
    Luminal.Log2 => 0, Luminal.Exp2 => 1, Luminal.Sin => 2, Luminal.Sqrt => 3, Luminal.Cos => 4, Luminal.Recip => 5,
    Luminal.Contiguous => 6, Luminal.ReLU => 7, Luminal.Add => 8, Luminal.Mul => 9, Luminal.Mod => 10, Luminal.Max => 11,
    Luminal.LessThan => 12, Luminal.FusedMulAdd => 13, Luminal.FusedAddReLU => 14, Luminal.MatMul => 15,
    Luminal.SumReduce => 16, Luminal.MaxReduce => 17, Luminal.Permute => 18, Luminal.Expand => 19, Luminal.Reshape => 20,
    Luminal.Slice => 21, Luminal.Pad => 22, Luminal.Unfold => 23, Luminal.Constant => 24, Luminal.FlashAttentionOp => 28)
const FUNCTION_CODES = Dict("InputTensor" => Int32(25), "Gather" => Int32(26), "CumSum" => Int32(27))
node_code(op::Luminal.Op) = get(NODE_CODES, typeof(op), Int32(29))
node_code(op::Luminal.Function) = get(FUNCTION_CODES, op.name, Int32(29))
node_args(::Luminal.Op) = Float64[]
node_args(op::Union{Luminal.SumReduce,Luminal.MaxReduce}) = Float64[op.dim]
node_args(op::Luminal.Permute) = Float64.(op.dims)
node_args(op::Luminal.Expand) = Float64[op.dim, op.size]
node_args(op::Luminal.Reshape) = Float64.(op.shape)
node_args(op::Luminal.Slice) = Float64[v for r in op.ranges for v in r]
node_args(op::Luminal.Pad) = Float64[v for r in op.padding for v in r]
node_args(op::Luminal.Unfold) = Float64[op.kernel_shape; op.stride_shape; op.dilation_shape]
node_args(op::Luminal.Constant) = Float64[op.value]
node_args(op::Luminal.FlashAttentionOp) = Float64[op.scale, op.causal]

# Graph.nodes and graph.tensors as the arrays lmb200_node_list and node_data point into; the caller keeps the result alive
function flatten(graph::Luminal.Graph)
    n = length(graph.nodes)
    op = Int32[node_code(nd.op) for nd in graph.nodes]
    in_off = Int32[0]; in_node = Int32[]; shape_off = Int32[0]; shape = Int64[]; arg_off = Int32[0]; arg = Float64[]
    for (nd, st) in zip(graph.nodes, graph.shapes)
        append!(in_node, Int32[i for (i, _, _) in nd.inputs]); push!(in_off, length(in_node))
        append!(shape, Int64.(Luminal.realized_dims(st))); push!(shape_off, length(shape))
        append!(arg, node_args(nd.op)); push!(arg_off, length(arg))
    end
    data = Ptr{Float32}[C_NULL for _ in 1:n]
    keep = Any[]
    for ((id, _), a) in graph.tensors
        a isa Array{Float32} || continue
        push!(keep, a); data[id] = pointer(a)
    end
    (n, op, in_off, in_node, shape_off, shape, arg_off, arg, data, keep)
end

function compile_b200(d::B200Device, graph::Luminal.Graph, output_id::Integer; dtype::Integer=F32, batch::Integer=0,
                      max_ctx::Integer=2048)
    flat = flatten(graph)
    n, op, in_off, in_node, shape_off, shape, arg_off, arg, data, _ = flat
    model = Ref{UInt64}(0); session = Ref{UInt64}(0); info = Ref(DecoderMatch(0, 0, 0, 0, 0, 0, 0, 0))
    GC.@preserve flat begin
        nl = NodeList(n, 0, pointer(op), pointer(in_off), pointer(in_node), pointer(shape_off), pointer(shape),
                      pointer(arg_off), pointer(arg))
        check(ccall((:lmb200_compile_node_list, LIB), Int32,
                    (UInt64, Ref{NodeList}, Int32, Ptr{Ptr{Float32}}, Int32, Int32, Int32, Int32, Ref{UInt64}, Ref{UInt64},
                     Ref{DecoderMatch}),
                    d.ctx, Ref(nl), output_id, data, COLMAJOR, dtype, batch, max_ctx, model, session, info))
    end
    vocab = Luminal.realized_dims(graph.shapes[output_id])[end]
    Model(model[]), Session(session[], batch > 0 ? batch : info[].batch, vocab), info[]
end

# The Whisper AudioEncoder (src/Whisper.jl:354-404) on the tensor cores.  compile_encoder_b200 recognises its graph
# (lmb200_compile_encoder_node_list; weights from graph.tensors as above) and returns the fused encoder; encode! runs a
# mel (batch, n_mels, frames) of any batch and length through it, cross_kv! projects the last output to every decoder
# layer's cross K/V inside a bf16 Whisper session (project_cross_kv, src/Whisper.jl:809-831, without the host).
struct EncoderMatch                                 # lmb200_encoder_match
    d_model::Int32; heads::Int32; layers::Int32; ffn::Int32; n_mels::Int32; batch::Int32; frames::Int32
    mel_node::Int32; rates_node::Int32; n_weights::Int32; eps::Float32
end
struct Encoder
    h::UInt64
    d_model::Int
end
function compile_encoder_b200(d::B200Device, graph::Luminal.Graph, output_id::Integer)
    flat = flatten(graph)
    n, op, in_off, in_node, shape_off, shape, arg_off, arg, data, _ = flat
    enc = Ref{UInt64}(0); info = Ref(EncoderMatch(0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0f0))
    GC.@preserve flat begin
        nl = NodeList(n, 0, pointer(op), pointer(in_off), pointer(in_node), pointer(shape_off), pointer(shape),
                      pointer(arg_off), pointer(arg))
        check(ccall((:lmb200_compile_encoder_node_list, LIB), Int32,
                    (UInt64, Ref{NodeList}, Int32, Ptr{Ptr{Float32}}, Int32, Ref{UInt64}, Ref{EncoderMatch}),
                    d.ctx, Ref(nl), output_id, data, COLMAJOR, enc, info))
    end
    Encoder(enc[], info[].d_model), info[]
end
function encode!(e::Encoder, mel::Array{Float32,3})
    batch, n_mels, frames = size(mel)
    rowmajor = permutedims(mel, (3, 2, 1))           # the entry takes the mel row-major: frames fastest
    out = Array{Float32}(undef, e.d_model, (frames - 1) ÷ 2 + 1, batch)
    check(ccall((:lmb200_whisper_encoder_run, LIB), Int32, (UInt64, Ptr{Float32}, Int32, Int32, Ptr{Float32}),
                e.h, rowmajor, batch, frames, out))
    permutedims(out, (3, 2, 1))                      # (batch, seq, d_model) as AudioEncoder returns it
end
cross_kv!(e::Encoder, s::Session) = check(ccall((:lmb200_whisper_encoder_cross_kv, LIB), Int32, (UInt64, UInt64), e.h, s.h))
destroy!(e::Encoder) = check(ccall((:lmb200_whisper_encoder_destroy, LIB), Int32, (UInt64,), e.h))

# tensor parallelism: one process per GPU; rank 0 creates the id, the launcher broadcasts the 128 bytes
function comm_unique_id()
    id = Vector{UInt8}(undef, 128)
    check(ccall((:lmb200_comm_unique_id, LIB), Int32, (Ptr{UInt8},), id))
    id
end
comm_init!(d::B200Device, n::Integer, rank::Integer, id::Vector{UInt8}) =
    check(ccall((:lmb200_comm_init, LIB), Int32, (UInt64, Int32, Int32, Ptr{UInt8}), d.ctx, n, rank, id))
comm_resync!(d::B200Device) = check(ccall((:lmb200_comm_resync, LIB), Int32, (UInt64,), d.ctx))
comm_destroy!(d::B200Device) = check(ccall((:lmb200_comm_destroy, LIB), Int32, (UInt64,), d.ctx))

end # module B200
