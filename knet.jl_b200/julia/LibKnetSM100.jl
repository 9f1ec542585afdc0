# LibKnetSM100.jl -- the Julia side of libknet_sm100.so.
#
# Drop-in for src/libknet8/LibKnet8.jl: the same `@knet8` / `@knet8r` macros, resolved
# against libknet_sm100.so, so every existing call site in src/knetarrays, src/cuarrays,
# src/ops20_gpu, src/ops21_gpu and src/autograd_gpu keeps working unchanged.  The second
# half adds methods that route the softmax family, nll, accuracy/argmax, dropout and
# update! to the fused entry points (section B of include/knet_sm100.h).
#
# This file could not be executed where the library was built (no Julia there); it is kept
# mechanically in step with the header: same names, same argument order.
module LibKnetSM100

export libknet8, @knet8, @knet8r

using CUDA, Libdl

# KNET_SM100_LIB overrides the search; otherwise look beside this file's package root.
const libknet8 = get(ENV, "KNET_SM100_LIB",
                     Libdl.find_library(["libknet_sm100"], [normpath(joinpath(@__DIR__, ".."))]))

"`@knet8(fun, (argtypes...), args...)`: call `fun_stream` on the task's CUDA stream."
macro knet8(fun, argtypes, args...)
    sym = string(fun isa QuoteNode ? fun.value : fun) * "_stream"
    if isa(argtypes, Expr) && argtypes.head == :tuple
        types = Expr(:tuple, argtypes.args..., :(CUDA.CUstream))
    else
        error("@knet8: argument types must be a tuple literal")
    end
    quote
        ccall(($sym, libknet8), Nothing, $(esc(types)), $(map(esc, args)...), CUDA.stream())
    end
end

"`@knet8r(fun, rettype, (argtypes...), args...)`: the value-returning form (synchronises)."
macro knet8r(fun, rettype, argtypes, args...)
    sym = string(fun isa QuoteNode ? fun.value : fun) * "_stream"
    types = Expr(:tuple, argtypes.args..., :(CUDA.CUstream))
    quote
        ccall(($sym, libknet8), $(esc(rettype)), $(esc(types)), $(map(esc, args)...), CUDA.stream())
    end
end

# ---------------------------------------------------------------------------------------
# Fused entry points.  `DevArray{T}` is Knet's Union{KnetArray{T},CuArray{T}}.
# ---------------------------------------------------------------------------------------
using Knet.KnetArrays: DevArray, KnetArray
using Knet.Ops20, Knet.Train20
using AutoGrad: AutoGrad, @primitive1, value

const STATUS = Dict(-1 => "invalid argument", -2 => "size not supported",
                    -3 => "workspace missing or too small", -4 => "pointer not aligned to its element size",
                    -5 => "NCCL could not be loaded", -6 => "timed out waiting for the other ranks",
                    -7 => "cuBLAS could not be loaded", -8 => "the loaded cuBLAS does not offer the requested mode")
check(rc, name) = rc == 0 ? nothing :
    error("$name: " * get(STATUS, rc, rc > 0 ? "CUDA error $rc" : "unknown error"))

# (inner, D, outer) of a run of adjacent dims; `nothing` when dims are not adjacent
function geometry(sz::Dims, dims)
    dims === Colon() && return (1, prod(sz), 1)
    ds = sort(unique(collect(dims)))
    ds == collect(ds[1]:ds[end]) || return nothing
    (prod(sz[1:ds[1]-1]), prod(sz[ds[1]:min(ds[end], length(sz))]), prod(sz[ds[end]+1:end]))
end

for (S, T) in ((32, Float32), (64, Float64))
    for (jl, fwd, bwd) in ((:_sm100_softmax, "knet_softmax_fwd_$S", "knet_softmax_bwd_$S"),
                           (:_sm100_logsoftmax, "knet_logsoftmax_fwd_$S", "knet_logsoftmax_bwd_$S"))
        jlback = Symbol(jl, :_back)
        @eval begin
            function $jl(x::DevArray{$T}; dims)
                g = geometry(size(x), dims); y = similar(x)
                check(ccall(($fwd, libknet8), Cint, (CuPtr{$T}, CuPtr{$T}, Int64, Int64, Int64, CUDA.CUstream),
                            x, y, g[1], g[2], g[3], CUDA.stream()), $fwd)
                y
            end
            function $jlback(y::DevArray{$T}, dy::DevArray{$T}; dims)
                g = geometry(size(y), dims); dx = similar(y)
                check(ccall(($bwd, libknet8), Cint, (CuPtr{$T}, CuPtr{$T}, CuPtr{$T}, Int64, Int64, Int64, CUDA.CUstream),
                            y, dy, dx, g[1], g[2], g[3], CUDA.stream()), $bwd)
                dx
            end
            @primitive1 $jl(x; dims), dy, y  $jlback(y, dy; dims=dims)
        end
    end
    lsef, lseb = "knet_logsumexp_fwd_$S", "knet_logsumexp_bwd_$S"
    nllf, nllb = "knet_nll_fwd_$S", "knet_nll_bwd_$S"
    amax, accf = "knet_argmax_$S", "knet_accuracy_$S"
    @eval begin
        function _sm100_logsumexp(x::DevArray{$T}; dims)
            g = geometry(size(x), dims)
            y = similar(x, ntuple(i -> (dims === Colon() || i in dims) ? 1 : size(x, i), ndims(x)))
            check(ccall(($lsef, libknet8), Cint, (CuPtr{$T}, CuPtr{$T}, Int64, Int64, Int64, CUDA.CUstream),
                        x, y, g[1], g[2], g[3], CUDA.stream()), $lsef)
            y
        end
        function _sm100_logsumexp_back(x::DevArray{$T}, y::DevArray{$T}, dy::DevArray{$T}; dims)
            g = geometry(size(x), dims); dx = similar(x)
            check(ccall(($lseb, libknet8), Cint,
                        (CuPtr{$T}, CuPtr{$T}, CuPtr{$T}, CuPtr{$T}, Int64, Int64, Int64, CUDA.CUstream),
                        x, y, dy, dx, g[1], g[2], g[3], CUDA.stream()), $lseb)
            dx
        end
        @primitive1 _sm100_logsumexp(x; dims), dy, y  _sm100_logsumexp_back(x, y, dy; dims=dims)

        # nll: labels go to the device once as Int32; total and count stay on the device
        # until the caller asks for the number.
        function _sm100_nll(scores::DevArray{$T}, labels::CuArray{Int32}; dims=1)
            R = size(scores, 1); K = div(length(scores), R)
            total = CUDA.zeros($T, 1); count = CUDA.zeros(Int32, 1)
            per = CuArray{$T}(undef, dims == 1 ? K : R)
            check(ccall(($nllf, libknet8), Cint,
                        (CuPtr{$T}, CuPtr{Int32}, Int64, Int64, Cint, CuPtr{$T}, CuPtr{Int32}, CuPtr{$T}, CUDA.CUstream),
                        scores, labels, R, K, dims, total, count, per, CUDA.stream()), $nllf)
            (total, count)
        end
        function _sm100_nll_back(scores::DevArray{$T}, labels::CuArray{Int32}, count::CuArray{Int32}, dy;
                                 dims=1, average=true)
            R = size(scores, 1); K = div(length(scores), R); dx = similar(scores)
            check(ccall(($nllb, libknet8), Cint,
                        (CuPtr{$T}, CuPtr{Int32}, Int64, Int64, Cint, Cint, $T, CuPtr{Int32}, CuPtr{$T}, CUDA.CUstream),
                        scores, labels, R, K, dims, average, $T(dy), count, dx, CUDA.stream()), $nllb)
            dx
        end
        function _sm100_argmax(x::DevArray{$T}; dims)
            g = geometry(size(x), dims); idx = CuArray{Int32}(undef, g[1] * g[3])
            check(ccall(($amax, libknet8), Cint, (CuPtr{$T}, CuPtr{Int32}, Int64, Int64, Int64, CUDA.CUstream),
                        x, idx, g[1], g[2], g[3], CUDA.stream()), $amax)
            idx
        end
        function _sm100_accuracy(scores::DevArray{$T}, labels::CuArray{Int32}; dims=1)
            R = size(scores, 1); K = div(length(scores), R); res = CUDA.zeros(Int32, 2)
            check(ccall(($accf, libknet8), Cint, (CuPtr{$T}, CuPtr{Int32}, Int64, Int64, Cint, CuPtr{Int32}, CUDA.CUstream),
                        scores, labels, R, K, dims, res, CUDA.stream()), $accf)
            Tuple(Array(res))
        end
        # A hidden layer h = dropout(relu.(w*x .+ b), p) as two fused calls: the forward writes h
        # over z = w*x with an in-kernel generator; the backward turns dh into dz in place
        # (dropback + reluback from h alone) and leaves db = sum(dz, dims=2) in the same pass.
        function _sm100_layer_fwd!(z::DevArray{$T}, b::DevArray{$T}, p::Real, seed::UInt64, offset::UInt64)
            N = length(b); B = div(length(z), N)
            check(ccall(($("knet_bias_relu_dropout_fwd_$S"), libknet8), Cint,
                        (CuPtr{$T}, CuPtr{$T}, CuPtr{$T}, Int64, Int64, $T, UInt64, UInt64, CUDA.CUstream),
                        z, b, z, N, B, $T(p), seed, offset, CUDA.stream()), "knet_bias_relu_dropout_fwd")
            z
        end
        function _sm100_layer_bwd!(h::DevArray{$T}, dh::DevArray{$T}, db::DevArray{$T}, p::Real)
            N = length(db); B = div(length(h), N)
            check(ccall(($("knet_relu_dropout_bias_bwd_$S"), libknet8), Cint,
                        (CuPtr{$T}, CuPtr{$T}, CuPtr{$T}, CuPtr{$T}, Int64, Int64, $T, CUDA.CUstream),
                        h, dh, dh, db, N, B, $T(p), CUDA.stream()), "knet_relu_dropout_bias_bwd")
            dh
        end
    end

    # update!: one ccall per optimizer (replaces the axpy!/lmul!/broadcast chains)
    for (opt, fn) in ((:SGD, "knet_sgd_$S"), (:Momentum, "knet_momentum_$S"), (:Adam, "knet_adam_$S"))
        if opt == :SGD
            @eval function Train20._update!(w::DevArray{$T}, g::DevArray{$T}, p::Train20.SGD)
                check(ccall(($fn, libknet8), Cint, (Int64, CuPtr{$T}, CuPtr{$T}, Cdouble, Cdouble, CUDA.CUstream),
                            length(w), w, g, p.lr, 1.0, CUDA.stream()), $fn)
                w
            end
        elseif opt == :Momentum
            @eval function Train20._update!(w::DevArray{$T}, g::DevArray{$T}, p::Train20.Momentum)
                p.velocity === nothing && (p.velocity = zero(w))
                check(ccall(($fn, libknet8), Cint,
                            (Int64, CuPtr{$T}, CuPtr{$T}, CuPtr{$T}, Cdouble, Cdouble, Cdouble, CUDA.CUstream),
                            length(w), w, g, p.velocity, p.lr, p.gamma, 1.0, CUDA.stream()), $fn)
                w
            end
        else
            @eval function Train20._update!(w::DevArray{$T}, g::DevArray{$T}, p::Train20.Adam)
                if p.fstm === nothing; p.fstm = zero(w); p.scndm = zero(w); end
                p.t += 1
                check(ccall(($fn, libknet8), Cint,
                            (Int64, CuPtr{$T}, CuPtr{$T}, CuPtr{$T}, CuPtr{$T}, Cdouble, Cdouble, Cdouble, Cdouble,
                             Cint, Cdouble, CUDA.CUstream),
                            length(w), w, g, p.fstm, p.scndm, p.lr, p.beta1, p.beta2, p.eps, p.t, 1.0, CUDA.stream()), $fn)
                w
            end
        end
    end
end

# Route Knet's user-facing functions to the fused kernels when dims are adjacent; anything
# else falls through to Knet's generic definitions (src/ops20/softmax.jl:42-70).
Ops20.softmax(x::DevArray; dims=:) =
    geometry(size(x), dims) === nothing ? Ops20._softmax(x; dims=dims) : _sm100_softmax(x; dims=dims)
Ops20.logsoftmax(x::DevArray; dims=:) =
    geometry(size(x), dims) === nothing ? Ops20._logsoftmax(x; dims=dims) : _sm100_logsoftmax(x; dims=dims)
Ops20.logsumexp(x::DevArray; dims=:) =
    geometry(size(x), dims) === nothing ? Ops20._logsumexp(x; dims=dims) : _sm100_logsumexp(x; dims=dims)

# ---- CuArray binary broadcast through the library --------------------------------------------
# Knet's vector/ND broadcast kernels are reached only from KnetArray methods
# (src/knetarrays/binary.jl:13-149); `x .+ b` on CuArrays goes to CUDA.jl's generic broadcast.
# KnetArray(::CuArray) shares the memory, so the CuArray forms can borrow the KnetArray dispatch
# (vbroadcast_shape, the _12/_13/_16 choice) and hand the result back as a CuArray.
for (f, op) in ((:+, "add"), (:-, "sub"), (:*, "mul"), (:/, "div"), (:max, "max"), (:min, "min"))
    @eval function Base.Broadcast.broadcasted(::typeof($f), x::CuArray{T}, y::CuArray{T}) where {T<:Union{Float32,Float64}}
        CuArray(Base.Broadcast.broadcasted($f, KnetArray(x), KnetArray(y)))
    end
end

# ---- data-parallel collectives (section C of knet_sm100.h): Knet has no counterpart -------------
# One process per GPU.  Rank 0 makes the id and hands it to the others out of band (a file, a
# socket, Distributed.jl); every rank then calls DpComm(id, rank, world) after CUDA.device!.
mutable struct DpComm
    handle::Ptr{Cvoid}
    rank::Int
    world::Int
end

function dp_unique_id()
    id = Vector{UInt8}(undef, 128)
    check(ccall((:knet_dp_unique_id, libknet8), Cint, (Ptr{UInt8},), id), :knet_dp_unique_id)
    id
end

function DpComm(id::Vector{UInt8}, rank::Integer, world::Integer; timeout_ms::Integer=60_000)
    h = Ref{Ptr{Cvoid}}(C_NULL)
    check(ccall((:knet_dp_init, libknet8), Cint, (Ptr{UInt8}, Cint, Cint, Cint, Ptr{Ptr{Cvoid}}),
                id, rank, world, timeout_ms, h), :knet_dp_init)      # status -6: a peer never joined
    DpComm(h[], rank, world)
end

for (T, S) in ((Float32, "32"), (Float64, "64"))
    ar, rs, ag = Symbol("knet_dp_allreduce_sum_", S), Symbol("knet_dp_reduce_scatter_sum_", S), Symbol("knet_dp_allgather_", S)
    @eval begin
        # sum of g over the ranks, in place; follow with update!(w, g .* (1/world)) or the fused gscale
        allreduce!(c::DpComm, g::DevArray{$T}) =
            (check(ccall(($(QuoteNode(ar)), libknet8), Cint, (Ptr{Cvoid}, CuPtr{$T}, Int64, CUDA.CUstream),
                         c.handle, g, length(g), CUDA.stream()), $(QuoteNode(ar))); g)
        # sharded update: recv has length(send) / world elements and may alias send's own part
        reduce_scatter!(c::DpComm, recv::DevArray{$T}, send::DevArray{$T}) =
            (check(ccall(($(QuoteNode(rs)), libknet8), Cint, (Ptr{Cvoid}, CuPtr{$T}, CuPtr{$T}, Int64, CUDA.CUstream),
                         c.handle, send, recv, length(recv), CUDA.stream()), $(QuoteNode(rs))); recv)
        allgather!(c::DpComm, recv::DevArray{$T}, send::DevArray{$T}) =
            (check(ccall(($(QuoteNode(ag)), libknet8), Cint, (Ptr{Cvoid}, CuPtr{$T}, CuPtr{$T}, Int64, CUDA.CUstream),
                         c.handle, send, recv, length(send), CUDA.stream()), $(QuoteNode(ag))); recv)
    end
end

Base.close(c::DpComm) = (check(ccall((:knet_dp_destroy, libknet8), Cint, (Ptr{Cvoid},), c.handle), :knet_dp_destroy); nothing)

# ---- matrix products (section D of knet_sm100.h) ----------------------------------------------------
# gemm!(transA, transB, alpha, A, B, beta, C) for KnetArray (src/knetarrays/linalg.jl:27-55) through
# knet_gemm_S_S: the same cuBLAS product, with GEMM_MODE[] = 1 asking cuBLAS (12.9 or later, e.g.
# KNET_SM100_CUBLAS_LIB pointing at it) for its FP32 emulation on the BF16 tensor cores.  One
# handle per task and device, as CUDA.jl's CUBLAS.handle(); the scratch is a KnetArray the caller
# may size with GEMM_WORKSPACE_MB.
const GEMM_MODE = Ref{Cint}(0)
const GEMM_WORKSPACE_MB = Ref{Int}(0)
mutable struct GemmHandle
    handle::Ptr{Cvoid}
    workspace::Union{Nothing,KnetArray{UInt8}}
end
function gemm_handle()
    get!(task_local_storage(), (:knet_sm100_gemm, CUDA.device())) do
        h = Ref{Ptr{Cvoid}}(C_NULL)
        check(ccall((:knet_gemm_create, libknet8), Cint, (Ptr{Ptr{Cvoid}},), h), :knet_gemm_create)
        ws = GEMM_WORKSPACE_MB[] > 0 ? KnetArray{UInt8}(undef, GEMM_WORKSPACE_MB[] << 20) : nothing
        g = GemmHandle(h[], ws)
        finalizer(x -> ccall((:knet_gemm_destroy, libknet8), Cint, (Ptr{Cvoid},), x.handle), g)
    end::GemmHandle
end
gemm_emulation_offered() = ccall((:knet_gemm_emulation, libknet8), Cint, (Ptr{Cvoid},), gemm_handle().handle) == 1

import LinearAlgebra.BLAS: gemm!
for (T, S) in ((Float32, "32"), (Float64, "64"))
    f = Symbol("knet_gemm_", S, "_S")
    @eval function gemm!(transA::AbstractChar, transB::AbstractChar, alpha::Number, A::KnetArray{$T},
                         B::KnetArray{$T}, beta::Number, C::KnetArray{$T})
        size2(x, i) = ndims(x) <= 2 ? size(x, i) : i == 1 ? div(length(x), size(x, ndims(x))) : size(x, ndims(x))
        ta, tb = transA != 'N', transB != 'N'
        m, k = ta ? (size2(A, 2), size2(A, 1)) : (size2(A, 1), size2(A, 2))
        n, kb = tb ? (size2(B, 1), size2(B, 2)) : (size2(B, 2), size2(B, 1))
        (k == kb && m == size2(C, 1) && n == size2(C, 2)) || throw(DimensionMismatch("$(map(size, (A, B, C)))"))
        g = gemm_handle()
        ws = g.workspace
        check(ccall(($(QuoteNode(f)), libknet8), Cint,
                    (Ptr{Cvoid}, Cint, Cint, Int64, Int64, Int64, $T, CuPtr{$T}, Int64, CuPtr{$T}, Int64, $T,
                     CuPtr{$T}, Int64, Cint, CuPtr{Cvoid}, Csize_t, CUDA.CUstream),
                    g.handle, ta, tb, m, n, k, alpha, A, size2(A, 1), B, size2(B, 1), beta, C, size2(C, 1),
                    $T === Float32 ? GEMM_MODE[] : 0, ws === nothing ? CU_NULL : pointer(ws),
                    ws === nothing ? 0 : length(ws), CUDA.stream()), $(QuoteNode(f)))
        C
    end
end

end # module
