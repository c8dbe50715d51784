# NOT EXECUTED: no Julia toolchain on the machines this repository was built and measured on.
#
# The reference has no GEMM bench script, only the test driver _run_ghb
# (test/gpu/blackwell/gemm_highperf_blackwell.jl:230-269). This is its twin for both backends:
# same operand packing (A as (K, M), B as (K, N) Julia arrays = [M,K] and [N,K] row-major), same
# CPU check (_ghb_cpu_ref, :224-228: bf16-quantised inputs, fp32 product, isapprox(rtol = atol = 5e-2)),
# plus a timing loop in the style of fab_time (bench/flash_attention.jl:109-135).
#
# Usage:  PTX_B200_NATIVE_LIB=/path/libptxb200.so PTX_GEMM_BACKEND=native julia --project bench/gemm.jl

using PTX, CUDACore, Test, Random

include(joinpath(@__DIR__, "..", "test", "setup.jl"))
# the kernel, its constants and _ghb_cpu_ref live in the test file (its testsets run once on include)
include(joinpath(@__DIR__, "..", "test", "gpu", "blackwell", "gemm_highperf_blackwell.jl"))

ghb_backend() = get(ENV, "PTX_GEMM_BACKEND", "dsl")

# One prepared problem: packed device operands, fp32 output, launch closure.
function ghb_setup(M, N, K; seed = 20260005)
    @assert M % 128 == 0 && N % 256 == 0 && K % 64 == 0
    rng = MersenneTwister(seed)
    A = Float32.(rand(rng, M, K)) .* 2f0 .- 1f0               # U[-1, 1], the full-size configuration's inputs
    B = Float32.(rand(rng, K, N)) .* 2f0 .- 1f0
    A_d = CuArray(BFloat16.(permutedims(A)))                   # (K, M): A row-major, K fastest
    Bt_d = CuArray(BFloat16.(B))                               # (K, N): B column-major = B^T row-major
    D_d = CUDACore.zeros(Float32, M * N)
    keep = Any[A_d, Bt_d]
    launch! = if ghb_backend() == "native"
        () -> PTX.gemm_native!(D_d, A_d, Bt_d, M, N, K; f32_out = true)
    else
        # the reference's own path, set up as _run_ghb does (gemm_highperf_blackwell.jl:249-263):
        # two tensor maps, their upload, and the one-tile-per-CTA kernel
        tmap_A = tensor_map_tile_2d(:bf16, pointer(A_d), M, K, GHB_BM, GHB_BK; swizzle = :B128)
        tmap_B = tensor_map_tile_2d(:bf16, pointer(Bt_d), N, K, GHB_BN, GHB_BK; swizzle = :B128)
        a_c = upload_tma_descriptor(tmap_A); b_c = upload_tma_descriptor(tmap_B)
        push!(keep, a_c, b_c)
        kern = @cuda launch=false _ghb_gemm_kernel!(D_d, a_c.ptr, b_c.ptr, Int32(M), Int32(N), Int32(K))
        CUDACore.attributes(kern.fun)[CUDACore.FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES] = GHB_SMEM
        () -> kern(D_d, a_c.ptr, b_c.ptr, Int32(M), Int32(N), Int32(K);
                   blocks = (N ÷ GHB_BN, M ÷ GHB_BM, 1), threads = GHB_THREADS, shmem = GHB_SMEM)
    end
    (; launch!, D_d, A, B, M, N, K, keepalive = keep)
end

function ghb_check(; M = 256, N = 512, K = 256)
    p = ghb_setup(M, N, K)
    p.launch!(); CUDACore.synchronize()
    got = permutedims(reshape(Array(p.D_d), N, M))             # D is [M, N] row-major
    ok = isapprox(got, _ghb_cpu_ref(p.A, p.B); rtol = 5e-2, atol = 5e-2)
    println("gemm check $(ghb_backend()): M=$M N=$N K=$K ", ok ? "OK" : "FAIL")
    ok
end

function ghb_time(; M = 8192, N = 8192, K = 8192, iters = 20, warmup = 3, warm_ms = 25.0)
    p = ghb_setup(M, N, K)
    t_warm = time_ns(); launches = 0
    while launches < warmup || (time_ns() - t_warm) < warm_ms * 1e6
        p.launch!(); launches += 1
    end
    CUDACore.synchronize()
    t0 = time_ns()
    for _ in 1:iters
        p.launch!()
    end
    CUDACore.synchronize()
    ms = (time_ns() - t0) / 1e6 / iters
    (; ms, tflops = 2.0 * M * N * K / (ms * 1e9))
end

if abspath(PROGRAM_FILE) == @__FILE__
    @assert ghb_check()
    r = ghb_time()
    println("$(ghb_backend()) gemm 8192^3: $(round(r.ms; digits = 4)) ms  $(round(r.tflops; digits = 1)) TFLOP/s")
end
