# TEST INFRASTRUCTURE, NOT EXECUTED: no Julia toolchain on the machines this repository was
# built on; kept so that a maintainer with Julia can check the C and numpy restatements
# (oracle/attention_oracle.c, oracle/oracle.py) against Julia's own arithmetic.
#
# Restatement of the reference's CPU checkers for the CPU-runnable configuration
# (B = 1, H = 4, S = 256, D = 64, non-causal, N(0,1) inputs, scale 1/8):
#   fab_cpu_ref   test/gpu/blackwell/flash_attention_defs.jl:967-976
#   fam_cpu_ref   test/gpu/ampere/flash_attention.jl:284-299  (causal: scores[r, c] = -Inf for c > r)
# Inputs are rounded to bf16 (round to nearest even), widened to Float32, and the output stays
# Float32. Reads the shared input files written by tests/golden/write_shared_inputs.py and
# writes its output beside them, for a byte-level comparison with the other oracles.

using BFloat16s

quantise(X) = Float32.(BFloat16.(X))

function attention_oracle(Q, K, V, sm_scale; causal = false)
    Qb, Kb, Vb = quantise(Q), quantise(K), quantise(V)
    scores = (Qb * Kb') .* Float32(sm_scale)
    if causal
        S = size(scores, 1)
        for c in 1:S, r in 1:(c - 1)
            scores[r, c] = -Inf32
        end
    end
    rmax = maximum(scores; dims = 2)
    ex = exp.(scores .- rmax)
    (ex ./ sum(ex; dims = 2)) * Vb
end

# bf16 bit patterns, [rows, D] row-major -> Float32 (rows, D)
function read_bits(path, rows, D)
    bits = Vector{UInt16}(undef, rows * D)
    read!(path, bits)
    permutedims(reshape(reinterpret(Float32, UInt32.(bits) .<< 16), D, rows))
end

function main(prefix; B = 1, H = 4, S = 256, D = 64, causal = false)
    Q = read_bits(prefix * "_q.bin", B * H * S, D)
    K = read_bits(prefix * "_k.bin", B * H * S, D)
    V = read_bits(prefix * "_v.bin", B * H * S, D)
    O = Matrix{Float32}(undef, B * H * S, D)
    for i in 1:(B * H)
        r = ((i - 1) * S + 1):(i * S)
        O[r, :] = attention_oracle(Q[r, :], K[r, :], V[r, :], 1f0 / sqrt(Float32(D)); causal)
    end
    write(prefix * "_o_julia_f32.bin", permutedims(O))          # row-major [rows, D] Float32
end

abspath(PROGRAM_FILE) == @__FILE__ && main(ARGS[1])
