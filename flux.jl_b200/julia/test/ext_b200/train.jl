# Mirrors test/train.jl:12-47, 89-94, 130-141 and test/ext_distributed/optimizer.jl:8-25 for the B200 device.
# NOT EXECUTED where this repository is built (no Julia toolchain).
using Test, Flux, B200Arrays, Optimisers, Random
const dev = B200Arrays.B200Device()

@testset "trainstep! semantics" begin
    m = Dense(reshape([0f0], 1, 1), false) |> dev
    opt = Flux.setup(Descent(0.1), m)
    x = dev(reshape([1f0], 1, 1))
    for _ in 1:50
        Flux.trainstep!((mm, xx) -> sum(mm(xx)), m, (x,), opt)
    end
    @test Flux.cpu(m).weight[1] ≈ -5 atol = 1e-4                                # test/train.jl:37-47
    l = Flux.trainstep!((mm, xx) -> sum(abs2, mm(xx)), m, (x,), opt)
    @test l ≈ 25 atol = 1e-3                                                    # the loss returned is pre-update (:89-94)
end

@testset "Adam on the device equals Adam on the host" begin
    Random.seed!(1)
    m = Chain(Dense(8 => 6, relu), Dense(6 => 3))
    md = m |> dev
    x, y = rand(Float32, 8, 16), Flux.onehotbatch(rand(1:3, 16), 1:3)
    xd, yd = dev(x), dev(Float32.(y))
    o, od = Flux.setup(Adam(1e-3), m), Flux.setup(Adam(1e-3), md)
    for _ in 1:5
        Flux.trainstep!((mm, a, b) -> Flux.logitcrossentropy(mm(a), b), m, (x, y), o)
        Flux.trainstep!((mm, a, b) -> Flux.logitcrossentropy(mm(a), b), md, (xd, yd), od)
    end
    @test Flux.cpu(md)[1].weight ≈ m[1].weight rtol = 1e-4 atol = 1e-5
end
