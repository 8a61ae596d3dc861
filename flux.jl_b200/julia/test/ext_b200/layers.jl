# Mirrors test/ext_cuda/layers.jl:15-27, 120-181, 343-363 of Flux for the B200 device: every hot-path layer, CPU (Zygote,
# the reference) against the same model moved to the device, outputs and gradients leaf by leaf with rtol = atol = 1e-4
# (test/test_module.jl:82-98).  Needs Julia, Flux, B200Arrays and a B200; NOT EXECUTED where this repository is built.
using Test, Flux, B200Arrays, Zygote, Random
using Flux: cpu
const dev = B200Arrays.B200Device()

function check_layer(m, x...; rtol=1f-4, atol=1f-4, loss=y -> sum(abs2, y isa Tuple ? first(y) : y))
    md = m |> dev
    xd = map(dev, x)
    y, yd = m(x...), md(xd...)
    @test isapprox(cpu(yd isa Tuple ? first(yd) : yd), y isa Tuple ? first(y) : y; rtol, atol)
    g = gradient(mm -> loss(mm(x...)), m)[1]
    gd = gradient(mm -> loss(mm(xd...)), md)[1]
    Flux.fmapstructure((a, b) -> a isa AbstractArray && @test(isapprox(cpu(b), a; rtol, atol)), g, gd)
    return nothing
end

@testset "Dense / Chain" begin
    Random.seed!(0)
    check_layer(Dense(10 => 5), rand(Float32, 10, 4))
    check_layer(Dense(10 => 5, relu), rand(Float32, 10, 4))
    check_layer(Dense(10 => 5, gelu; bias=false), rand(Float32, 10, 4))
    check_layer(Chain(Dense(784 => 512, relu), Dense(512 => 512, relu), Dense(512 => 10)), rand(Float32, 784, 64))
    check_layer(Dense(10 => 5), rand(Float32, 10, 3, 2))                        # N-d input (basic.jl:202-205)
    # ones-init known answers (test/layers/basic.jl:85-89)
    @test cpu((Dense(10 => 1; init=ones) |> dev)(dev(ones(Float32, 10, 1)))) == 10 * ones(1, 1)
    @test cpu((Dense(10 => 2; init=ones) |> dev)(dev([ones(Float32, 10, 1) 2 * ones(Float32, 10, 1)]))) == [10 20; 10 20]
    # no bias: its gradient is nothing (test/ext_cuda/layers.jl:120-127)
    d = Dense(10 => 5; bias=false) |> dev
    @test gradient(m -> sum(abs2, m(dev(rand(Float32, 10, 2)))), d)[1].bias === nothing
    @test_throws DimensionMismatch d(dev(rand(Float32, 11, 2)))
end

@testset "normalisation" begin
    check_layer(LayerNorm(16), rand(Float32, 16, 8))
    check_layer(LayerNorm(16, tanh), rand(Float32, 16, 8))
    check_layer(Flux.trainmode!(BatchNorm(4, relu)), rand(Float32, 5, 5, 4, 3))
    check_layer(GroupNorm(4, 2), rand(Float32, 5, 5, 4, 3))
    check_layer(Flux.trainmode!(InstanceNorm(4; affine=true)), rand(Float32, 5, 5, 4, 3))
    # statistics are tracked only in gradient / train mode (test/ext_cuda/layers.jl:129-181)
    bn = BatchNorm(2) |> dev
    x = dev(Float32[1 3 5; 2 4 6])
    bn(x); @test cpu(bn.μ) == [0, 0]
    gradient(m -> sum(abs2, m(x)), bn); @test cpu(bn.μ) ≈ [0.3, 0.4]
    @test cpu(bn.σ²) ≈ [1.3, 1.3]
    @test_throws ArgumentError Flux.trainmode!(BatchNorm(2) |> dev)(dev(rand(Float32, 2, 1)))
    # frozen GroupNorm literal (test/layers/normalisation.jl:410)
    y = cpu((GroupNorm(4, 2) |> dev)(dev(Float32.(reshape(1:24, 3, 4, 2)))))
    @test y[:, :, 1] ≈ [-1.4638476 0.29276943 -1.4638476 0.29276943; -0.87830865 0.87830853 -0.8783088 0.8783083; -0.29276967 1.4638474 -0.2927699 1.4638472] atol = 1e-5
end

@testset "recurrent" begin
    for cell in (LSTMCell(3 => 5), GRUCell(3 => 5), RNNCell(3 => 5), Flux.GRUv3Cell(3 => 5))
        check_layer(Recurrence(cell), rand(Float32, 3, 7, 4))
    end
    lstm = LSTM(3 => 5) |> dev
    x = dev(rand(Float32, 3, 7, 4))
    @test size(lstm(x)) == (5, 7, 4)
    @test cpu((Recurrence(lstm.cell; return_state=true))(x)[2][1]) ≈ cpu(lstm(x))[:, end, :]
end

@testset "MultiHeadAttention" begin
    mha = MultiHeadAttention(16, nheads=2)
    x = rand(Float32, 16, 9, 3)
    mask = NNlib.make_causal_mask(x)
    check_layer(mha, x; loss=y -> sum(abs2, first(y)))
    md, xd = mha |> dev, dev(x)
    y, α = md(xd; mask)
    yc, αc = mha(x; mask)
    @test cpu(y) ≈ yc atol = 1e-4                                              # test/ext_cuda/layers.jl:343-363
    @test Array(α) ≈ αc atol = 1e-4
    @test all(Array(α)[2, 1, :, :] .== 0)                                       # test/layers/attention.jl:38-43
end

@testset "Embedding / Dropout" begin
    emb = Embedding(26 => 4) |> dev
    idx = dev([3, 1, 20, 14, 4, 15, 7])
    @test cpu(emb(idx)) == cpu(emb).weight[:, [3, 1, 20, 14, 4, 15, 7]]
    d = Flux.trainmode!(Dropout(0.5))
    y = cpu(d(dev(ones(Float32, 1000))))
    @test all(v -> v == 0 || v == 2, y) && 350 < count(==(0), y) < 650       # test/layers/normalisation.jl:10-30
    @test cpu(Flux.testmode!(Dropout(0.5))(dev(ones(Float32, 10)))) == ones(10)
end
