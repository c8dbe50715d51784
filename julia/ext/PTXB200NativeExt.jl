# NOT EXECUTED: neither the machine this was written on nor the GPU boxes it was measured on
# have a Julia toolchain. Reviewed as code against the C ABI in include/ptxb200.h only.
#
# Package extension for jool-space/PTX.jl that routes the flash-attention forward pass, the
# bf16 GEMMs and the row-wise kernels to libptxb200.so (hand-written CUDA for sm_100a) through
# ccall. It sits beside ext/CUDACoreExt.jl and is triggered by the same weak dependency:
#
#   Project.toml   [extensions]  PTXB200NativeExt = "CUDACore"        (next to CUDACoreExt, :15-20)
#   src/PTX.jl     function fa_fwd_native! end; function gemm_native! end; function gemm_grouped_native! end
#                  function softmax_native! end; function rms_norm_native! end; function layer_norm_native! end
#                  function swiglu_native! end; function native_status end; function fa_fwd_noalloc! end
#                  (stub generics; the methods come from this file, as src/lib/tensor_map.jl:147,160,201 does
#                  for the tensor-map functions)
#
# The library is found through ENV["PTX_B200_NATIVE_LIB"]. Arrays keep the reference's layout:
# Q, K, V, O as CuArray{BFloat16} of size (D, B*H*S) -- fab_pack's output, i.e. [B,H,S,D] row-major
# (test/gpu/blackwell/flash_attention_defs.jl:979-986); GEMM A as (K, M), B as (K, N).
module PTXB200NativeExt

using PTX
using CUDACore: CUDACore, CuArray, CuPtr
using Libdl

const LIB = Ref{Ptr{Cvoid}}(C_NULL)

function lib()
    if LIB[] == C_NULL
        path = get(ENV, "PTX_B200_NATIVE_LIB", "")
        isempty(path) && error("PTX_B200_NATIVE_LIB is not set (path to libptxb200.so)")
        LIB[] = Libdl.dlopen(path)
    end
    LIB[]
end

sym(name) = Libdl.dlsym(lib(), name)

function check(rc::Cint)
    rc == 0 && return nothing
    msg = unsafe_string(ccall(sym(:ptxb200_strerror), Cstring, (Cint,), rc))
    detail = unsafe_string(ccall(sym(:ptxb200_last_cuda_error), Cstring, ()))
    error("ptxb200: $msg $(isempty(detail) ? "" : "-- " * detail)")
end

stream_handle() = reinterpret(Ptr{Cvoid}, CUDACore.stream().handle)

# O, Q, K, V :: CuArray{BFloat16} holding (D, B*H*S); same layout as fab_pack's output.
function PTX.fa_fwd_native!(O::CuArray, Q::CuArray, K::CuArray, V::CuArray,
                            B::Integer, H::Integer, S::Integer, D::Integer;
                            sm_scale::Real = 1 / sqrt(Float32(D)), causal::Bool = false,
                            flags::Integer = 0)
    GC.@preserve O Q K V begin
        rc = ccall(sym(:fa_fwd_bf16), Cint,
                   (CuPtr{Cvoid}, CuPtr{Cvoid}, CuPtr{Cvoid}, CuPtr{Cvoid},
                    Cint, Cint, Cint, Cint, Cfloat, Cint, Cuint, CuPtr{Cvoid}, Ptr{Cvoid}),
                   pointer(O), pointer(Q), pointer(K), pointer(V),
                   B, H, S, D, Float32(sm_scale), causal ? 1 : 0, flags,
                   CUDACore.CU_NULL, stream_handle())
    end
    check(rc)
    O
end

# C (M*N, bf16 or fp32), A packed (K, M), Bt packed (K, N) as in _run_ghb.
function PTX.gemm_native!(C::CuArray, A::CuArray, Bt::CuArray, M::Integer, N::Integer, K::Integer;
                          f32_out::Bool = eltype(C) == Float32)
    GC.@preserve C A Bt begin
        rc = ccall(sym(:gemm_bf16), Cint,
                   (CuPtr{Cvoid}, CuPtr{Cvoid}, CuPtr{Cvoid}, Cint, Cint, Cint, Cint, Cuint, Ptr{Cvoid}),
                   pointer(C), pointer(A), pointer(Bt), M, N, K, N, f32_out ? 1 : 0, stream_handle())
    end
    check(rc)
    C
end

# Uniform grouped GEMM: A packed (K, G*M), Bt packed (K, G*N) as _ggb_pack_A/_ggb_pack_B, C (G*M*N).
function PTX.gemm_grouped_native!(C::CuArray, A::CuArray, Bt::CuArray, G::Integer, M::Integer,
                                  N::Integer, K::Integer; f32_out::Bool = eltype(C) == Float32)
    GC.@preserve C A Bt begin
        rc = ccall(sym(:gemm_bf16_grouped), Cint,
                   (CuPtr{Cvoid}, CuPtr{Cvoid}, CuPtr{Cvoid}, Cint, Cint, Cint, Cint, Cint, Cuint, Ptr{Cvoid}),
                   pointer(C), pointer(A), pointer(Bt), G, M, N, K, N, f32_out ? 1 : 0, stream_handle())
    end
    check(rc)
    C
end

# Row-wise fp32 kernels on flat row-major vectors (element (b, i) at b*N + i), as the
# reference's testsets pass them.
function PTX.softmax_native!(Y::CuArray{Float32}, X::CuArray{Float32}, rows::Integer, N::Integer)
    GC.@preserve Y X check(ccall(sym(:softmax_f32), Cint,
        (CuPtr{Cvoid}, CuPtr{Cvoid}, Cint, Cint, Ptr{Cvoid}), pointer(Y), pointer(X), rows, N, stream_handle()))
    Y
end
function PTX.rms_norm_native!(Y::CuArray{Float32}, X::CuArray{Float32}, W::CuArray{Float32},
                              rows::Integer, N::Integer, eps::Real)
    GC.@preserve Y X W check(ccall(sym(:rms_norm_f32), Cint,
        (CuPtr{Cvoid}, CuPtr{Cvoid}, CuPtr{Cvoid}, Cint, Cint, Cfloat, Ptr{Cvoid}),
        pointer(Y), pointer(X), pointer(W), rows, N, Float32(eps), stream_handle()))
    Y
end
function PTX.layer_norm_native!(Y::CuArray{Float32}, X::CuArray{Float32}, W::CuArray{Float32},
                                Bias::CuArray{Float32}, rows::Integer, N::Integer, eps::Real)
    GC.@preserve Y X W Bias check(ccall(sym(:layer_norm_f32), Cint,
        (CuPtr{Cvoid}, CuPtr{Cvoid}, CuPtr{Cvoid}, CuPtr{Cvoid}, Cint, Cint, Cfloat, Ptr{Cvoid}),
        pointer(Y), pointer(X), pointer(W), pointer(Bias), rows, N, Float32(eps), stream_handle()))
    Y
end
function PTX.swiglu_native!(out::CuArray{Float32}, gate::CuArray{Float32}, up::CuArray{Float32})
    GC.@preserve out gate up check(ccall(sym(:swiglu_f32), Cint,
        (CuPtr{Cvoid}, CuPtr{Cvoid}, CuPtr{Cvoid}, Clonglong, Ptr{Cvoid}),
        pointer(out), pointer(gate), pointer(up), length(gate), stream_handle()))
    out
end

# Synchronises the task-local stream; 0 = healthy, otherwise throws with the decoded site.
function PTX.native_status()
    rc = ccall(sym(:ptxb200_sync_status), Cint, (Ptr{Cvoid},), stream_handle())
    rc == 0 || check(rc)
    rc
end


# fa_fwd_native! without any device allocation by the library (its scratch is a 1 KiB array in
# the library image): for sessions where every byte on the GPU must come from CUDA.jl's pool.
# Non-causal calls need S % 128 == 0. Check with native_noalloc_status().
function PTX.fa_fwd_noalloc!(O::CuArray, Q::CuArray, K::CuArray, V::CuArray,
                             B::Integer, H::Integer, S::Integer, D::Integer;
                             sm_scale::Real = 1 / sqrt(Float32(D)), causal::Bool = false,
                             flags::Integer = 0)
    GC.@preserve O Q K V begin
        rc = ccall(sym(:fa_fwd_bf16_noalloc), Cint,
                   (CuPtr{Cvoid}, CuPtr{Cvoid}, CuPtr{Cvoid}, CuPtr{Cvoid},
                    Cint, Cint, Cint, Cint, Cfloat, Cint, Cuint, Ptr{Cvoid}),
                   pointer(O), pointer(Q), pointer(K), pointer(V),
                   B, H, S, D, Float32(sm_scale), causal ? 1 : 0, flags, stream_handle())
    end
    check(rc)
    O
end

function native_noalloc_status()
    flags = zeros(UInt32, 240)
    rc = ccall(sym(:fa_fwd_bf16_noalloc_status), Cint, (Ptr{UInt32}, Cint, Ptr{Cvoid}),
               flags, length(flags), stream_handle())
    rc == 0 || check(rc)
    rc
end

end # module
