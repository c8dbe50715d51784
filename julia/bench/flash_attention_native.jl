# NOT EXECUTED: no Julia toolchain on the machines this repository was built and measured on.
#
# Twin of bench/flash_attention.jl for the native backend. It includes the reference's own
# driver (so fab_check, fab_time, fab_sweep and fab_cpu_ref are the reference's, unchanged) and
# then redefines fab_setup with the ONE difference the backend swap needs: the launch closure.
# In the reference's file the same swap is one line, replacing bench/flash_attention.jl:78-82:
#
#     launch! = get(ENV, "PTX_FA_BACKEND", "dsl") == "native" ?
#         (() -> PTX.fa_fwd_native!(O_d, Q_d, K_d, V_d, B, H, S, FAB_HD; sm_scale)) :
#         (() -> kern(args...; blocks = (num_ctas, 1, 1), threads = FAB_THREADS, shmem = FAB_SMEM_BYTES))
#
# Usage:  PTX_B200_NATIVE_LIB=/path/libptxb200.so julia --project bench/flash_attention_native.jl
#         PTX_FA_INPUTS=/path/prefix  -> Q, K, V are read from <prefix>_{q,k,v}.bin (bf16 bits,
#         [B*H*S, D] row-major, written by tests/golden/write_shared_inputs.py) instead of being
#         drawn from MersenneTwister, so that both backends and the Python harness see the same bytes.

include(joinpath(@__DIR__, "flash_attention.jl"))   # the reference driver: fab_check, fab_time, fab_sweep, ...

# bf16 bit patterns on disk -> Float32 matrix (rows, FAB_HD), the type fab_setup keeps for fab_cpu_ref
function fab_read_bits(path, rows)
    bits = Vector{UInt16}(undef, rows * FAB_HD)
    read!(path, bits)
    f = reinterpret(Float32, UInt32.(bits) .<< 16)
    permutedims(reshape(f, FAB_HD, rows))          # file is row-major [rows, HD]
end

# Same signature and same returned NamedTuple as the reference's fab_setup
# (bench/flash_attention.jl:41-85); no tensor maps, no descriptor upload, no JIT of fab_kernel!.
function fab_setup(B, H, S; input_scale = 0.5f0, cfg = FAB_CFG_DEFAULT)
    bh = B * H
    total_rows = bh * S
    sm_scale = 1.0f0 / sqrt(Float32(FAB_HD))
    prefix = get(ENV, "PTX_FA_INPUTS", "")
    if isempty(prefix)
        rng = MersenneTwister(B * 7919 + H * 131 + S)
        Q = Float32.(randn(rng, total_rows, FAB_HD)) .* input_scale
        K = Float32.(randn(rng, total_rows, FAB_HD)) .* input_scale
        V = Float32.(randn(rng, total_rows, FAB_HD))
    else
        Q = fab_read_bits(prefix * "_q.bin", total_rows)
        K = fab_read_bits(prefix * "_k.bin", total_rows)
        V = fab_read_bits(prefix * "_v.bin", total_rows)
    end
    Q_d = CuArray(fab_pack(Q)); K_d = CuArray(fab_pack(K)); V_d = CuArray(fab_pack(V))
    O_d = CUDACore.zeros(BFloat16, total_rows * FAB_HD)
    dbg_d = CUDACore.zeros(UInt32, FAB_THREADS)
    n_sms = CUDACore.attribute(CUDACore.device(), CUDACore.DEVICE_ATTRIBUTE_MULTIPROCESSOR_COUNT)
    num_ctas = min(cld(S, 256) * bh, n_sms)
    launch! = () -> PTX.fa_fwd_native!(O_d, Q_d, K_d, V_d, B, H, S, FAB_HD; sm_scale)
    (; launch!, O_d, dbg_d, Q, K, V, sm_scale, B, H, S, num_ctas, keepalive = (Q_d, K_d, V_d))
end

if abspath(PROGRAM_FILE) == @__FILE__
    @assert fab_check()                                   # rescale-heavy inputs, the reference's gate (5e-2)
    @assert fab_check(; B = 2, H = 4, S = 1024, input_scale = 0.5f0)
    r = fab_time(; B = 4, H = 16, S = 4096)               # the headline configuration
    println("native fa_fwd_bf16: B=4 H=16 S=4096 D=$(FAB_HD)  $(round(r.ms; digits = 4)) ms  ",
            "$(round(r.tflops; digits = 1)) TFLOP/s  ctas=$(r.ctas)")
    PTX.native_status()
end
