# Julia glue that puts libevotrees_b200.so behind EvoTrees' `device = :gpu` dispatch points, in place of
# ext/EvoTreesCUDAExt.jl + ext/EvoTreesKernelAbstractionsExt/.  It needs neither CUDA.jl nor KernelAbstractions:
# every device operation is a `ccall` into the C ABI of include/evb.h.
#
# NOT EXECUTED in the build image (no Julia runtime there): this file is the binding a maintainer adds; the
# same call sequence is exercised by the Python mirror of this package (fit.py / model.py).
#
# Load order: `using EvoTrees; include("EvoTreesB200Ext.jl")` with ENV["EVOTREES_B200_LIB"] pointing at the
# shared library.  Do not load CUDA.jl's extension at the same time (both attach to `CUDADevice`).
module EvoTreesB200Ext

using EvoTrees
using EvoTrees: CUDADevice, GPU, CacheGPU, EvoTree, Tree, EvoTypes, _init_target, get_edges, binarize, _loss2type_dict
using Random: Xoshiro, rand!
using StatsBase: sample!

const LIB = get(ENV, "EVOTREES_B200_LIB", "libevotrees_b200.so")

# evb_params (include/evb.h); field order and types must match the C struct
struct EvbParams
    loss::Int32; K::Int32; nbins::Int32; max_depth::Int32; bagging_size::Int32; tree_type::Int32
    eta::Float64; lambda::Float64; L2::Float64; gamma::Float64; min_weight::Float64
    device::Int32; flags::UInt32
    alpha::Float64
    alphas::NTuple{8,Float64}
end

const LOSS_CODE = Dict(:mse => 0, :logloss => 1, :mlogloss => 2, :gaussian_mle => 3, :poisson => 4, :gamma => 5, :tweedie => 6, :logistic_mle => 7,
    :mae => 8, :cred_var => 9, :cred_std => 10, :quantile => 11, :multiquantile => 12)
# loss type of a fitted model (the `L` of `EvoTree{L,K}`) -> code: the inverse of the reference's own table (src/loss.jl:20-34)
const LOSS_TYPE_CODE = Dict(T => LOSS_CODE[s] for (s, T) in _loss2type_dict)

function check(rc::Int32)
    rc == 0 && return nothing
    error(unsafe_string(ccall((:evb_last_error, LIB), Cstring, ())))
end

# Counterpart of CacheBaseGPU (ext/EvoTreesKernelAbstractionsExt/structs.jl): the device state lives behind `handle`.
mutable struct B200Cache <: CacheGPU
    handle::Ptr{Cvoid}
    rng::Xoshiro
    K::Int
    nobs::Int
    mask_cpu::Vector{UInt8}
    mask_cond::UInt8
    js_::Vector{UInt32}
    js::Vector{UInt32}
    feature_names::Vector{Symbol}
    feattypes::Vector{Bool}
    function B200Cache(args...)
        c = new(args...)
        finalizer(c -> (c.handle != C_NULL && ccall((:evb_destroy, LIB), Cvoid, (Ptr{Cvoid},), c.handle); c.handle = C_NULL), c)
        return c
    end
end

# hooks that `init` / `fit` call on the device type (src/init.jl:300-301, src/fit.jl:266)
EvoTrees.device_ones(::Type{<:GPU}, ::Type{T}, n::Int) where {T} = ones(T, n)
EvoTrees.device_array_type(::Type{<:GPU}) = Array          # host arrays: the upload happens inside evb_create
EvoTrees.post_fit_gc(::Type{<:GPU}) = nothing              # the handle outlives `fit` (MLJ `update` resumes on it)

# Device blocks of destroyed handles and of finished inference calls stay with the library for reuse; this hands them
# back to the driver (what `GC.gc(); CUDA.reclaim()` is for CUDA.jl's pool in the reference's post_fit_gc).
trim_cache(device::Integer=0) = check(ccall((:evb_trim_cache, LIB), Int32, (Int32,), Int32(device)))

# replaces ext/EvoTreesKernelAbstractionsExt/init.jl:1-151
function EvoTrees.init_core(params::EvoTypes, ::Type{<:GPU}, data, feature_names, y_train, w, offset)
    params.tree_type in (:binary, :oblivious) || error("EvoTreesB200Ext: tree_type must be :binary or :oblivious")
    haskey(LOSS_CODE, params.loss) || error("EvoTreesB200Ext supports losses $(collect(keys(LOSS_CODE)))")
    rng = Xoshiro(params.seed)
    edges, featbins, feattypes = get_edges(data; feature_names, nbins=params.nbins, rng)   # same RNG stream as the CPU path
    # A dense Float32 / Float64 matrix is binarized on the device (evb_create_x below); anything else (a table, mixed
    # column types, categorical columns) goes through the reference's own `binarize` and travels as bins.
    raw = data isa Matrix{Float32} || data isa Matrix{Float64}
    x_bin = raw ? nothing : binarize(data; feature_names, edges)                           # Matrix{UInt8}, column-major
    nobs, nfeats = raw ? size(data) : size(x_bin)
    T = Float32
    L = _loss2type_dict[params.loss]
    K, y, μ, target_levels, target_isordered = _init_target(L, y_train, params, offset, T)
    !isnothing(offset) && (μ .= 0)
    @assert (size(y, ndims(y)) == length(w) && minimum(w) > 0)
    pred0 = zeros(T, K, nobs); pred0 .= μ
    !isnothing(offset) && (pred0 .+= offset')
    monotone = zeros(Int32, nfeats)
    hasproperty(params, :monotone_constraints) && for (k, v) in params.monotone_constraints
        monotone[k] = v
    end
    p = Ref(EvbParams(LOSS_CODE[params.loss], K, params.nbins, params.max_depth, params.bagging_size, params.tree_type == :oblivious ? 1 : 0,
        params.eta, params.lambda, params.L2, params.gamma, params.min_weight, 0, 0,
        hasproperty(params, :alpha) ? Float64(params.alpha) : 0.5,
        ntuple(k -> hasproperty(params, :alphas) && k <= length(params.alphas) ? Float64(params.alphas[k]) : 0.0, 8)))
    ydt, ycols = y isa Vector{UInt32} ? (Int32(1), Int32(1)) : (Int32(0), Int32(ndims(y) == 1 ? 1 : size(y, 1)))
    handle = Ref{Ptr{Cvoid}}(C_NULL)
    ft = UInt8.(feattypes)
    if raw
        E = eltype(data)
        edges_mat = reduce(hcat, [E.(e) for e in edges])                                   # [nbins - 1, nfeats], column-major
        GC.@preserve data edges_mat y w pred0 ft monotone check(ccall((:evb_create_x, LIB), Int32,
            (Ref{Ptr{Cvoid}}, Ref{EvbParams}, Int64, Int32, Ptr{Cvoid}, Int32, Ptr{Cvoid}, Int32, Ptr{Cvoid}, Int32, Int32, Ptr{Float32}, Ptr{Float32}, Ptr{Float32}, Ptr{UInt8}, Ptr{Int32}),
            handle, p, nobs, nfeats, data, E == Float32 ? 0 : 2, edges_mat, size(edges_mat, 1), y, ydt, ycols, w, pred0, C_NULL, ft, monotone))
    else
        GC.@preserve x_bin y w pred0 ft monotone check(ccall((:evb_create, LIB), Int32,
            (Ref{Ptr{Cvoid}}, Ref{EvbParams}, Int64, Int32, Ptr{UInt8}, Ptr{Cvoid}, Int32, Int32, Ptr{Float32}, Ptr{Float32}, Ptr{Float32}, Ptr{UInt8}, Ptr{Int32}),
            handle, p, nobs, nfeats, x_bin, y, ydt, ycols, w, pred0, C_NULL, ft, monotone))
    end
    info = Dict(:nrounds => 0, :feature_names => feature_names, :target_levels => target_levels,
        :target_isordered => target_isordered, :edges => edges, :featbins => featbins, :feattypes => feattypes)
    m = EvoTree{L,K}(L, K, [Tree{L,K}(μ)], info)
    js = zeros(UInt32, ceil(Int, params.colsample * nfeats))
    cache = B200Cache(handle[], rng, K, nobs, zeros(UInt8, nobs), round(UInt8, 255 * params.rowsample),
        collect(UInt32(1):UInt32(nfeats)), js, feature_names, feattypes)
    LAST_CACHE[] = cache   # read by the CallBack constructor below
    return m, cache
end

# replaces ext/EvoTreesKernelAbstractionsExt/fit.jl:1-21 (and everything it calls)
function EvoTrees.grow_evotree!(m::EvoTree{L,K}, cache::B200Cache, params::EvoTypes) where {L,K}
    for bag in 1:params.bagging_size
        rand!(cache.rng, cache.mask_cpu)                                              # same draws as subsample()
        sample!(cache.rng, cache.js_, cache.js, replace=false, ordered=true)
        tree = Tree{L,K}(params.max_depth)
        split8 = zeros(UInt8, length(tree.split))
        GC.@preserve tree split8 check(ccall((:evb_grow_tree, LIB), Int32,
            (Ptr{Cvoid}, Ptr{UInt8}, UInt8, Ptr{UInt32}, Int32, Int32, Ptr{Int64}, Ptr{UInt8}, Ptr{Float32}, Ptr{Float32}, Ptr{Float32}, Ptr{UInt8}),
            cache.handle, params.rowsample < 1 ? pointer(cache.mask_cpu) : Ptr{UInt8}(C_NULL), cache.mask_cond, cache.js,
            length(cache.js), bag == 1 ? 1 : 0, tree.feat, tree.cond_bin, tree.w, tree.gain, tree.pred, split8))
        tree.split .= split8 .!= 0
        push!(m.trees, tree)
    end
    m.info[:nrounds] += 1
    return nothing
end

function pack(m::EvoTree{L,K}, ntree_limit) where {L,K}
    nn = maximum(length(t.feat) for t in m.trees[1:ntree_limit])
    feat = zeros(Int64, nn, ntree_limit); cb = zeros(UInt8, nn, ntree_limit); sp = zeros(UInt8, nn, ntree_limit)
    lp = zeros(Float32, K, nn, ntree_limit)
    for (i, t) in enumerate(m.trees[1:ntree_limit])
        k = length(t.feat)
        feat[1:k, i] .= t.feat; cb[1:k, i] .= t.cond_bin; sp[1:k, i] .= t.split; lp[:, 1:k, i] .= t.pred
    end
    return nn, feat, cb, sp, lp
end

# replaces ext/EvoTreesKernelAbstractionsExt/predict.jl:115-135
function EvoTrees._predict(m::EvoTree{L,K}, data, ::Type{<:GPU}; ntree_limit=length(m.trees)) where {L,K}
    ntree_limit > length(m.trees) && error("ntree_limit is larger than number of trees $(length(m.trees)).")
    x_bin = binarize(data; feature_names=m.info[:feature_names], edges=m.info[:edges])
    nobs, nfeats = size(x_bin)
    nn, feat, cb, sp, lp = pack(m, ntree_limit)
    out = zeros(Float32, nobs, K)
    ft = UInt8.(m.info[:feattypes])
    code = LOSS_TYPE_CODE[L]
    GC.@preserve x_bin feat cb sp lp ft out check(ccall((:evb_predict, LIB), Int32,
        (Int32, Int32, Int32, Int32, Int32, Ptr{Int64}, Ptr{UInt8}, Ptr{UInt8}, Ptr{Float32}, Ptr{UInt8}, Int64, Int32, Ptr{UInt8}, Int32, Ptr{Float32}, Ptr{UInt32}),
        0, code, K, ntree_limit, nn, feat, cb, sp, lp, x_bin, nobs, nfeats, ft, 1, out, C_NULL))
    return K == 1 ? vec(out) : out
end

# replaces ext/EvoTreesKernelAbstractionsExt/predict.jl:138-158
function EvoTrees._predict_leaf_indices(m::EvoTree{L,K}, data, ::Type{<:GPU}; ntree_limit=length(m.trees)) where {L,K}
    x_bin = binarize(data; feature_names=m.info[:feature_names], edges=m.info[:edges])
    nobs, nfeats = size(x_bin)
    nn, feat, cb, sp, lp = pack(m, ntree_limit)
    out = zeros(Float32, nobs, K); leaf = zeros(UInt32, nobs, ntree_limit)
    ft = UInt8.(m.info[:feattypes])
    GC.@preserve x_bin feat cb sp lp ft out leaf check(ccall((:evb_predict, LIB), Int32,
        (Int32, Int32, Int32, Int32, Int32, Ptr{Int64}, Ptr{UInt8}, Ptr{UInt8}, Ptr{Float32}, Ptr{UInt8}, Int64, Int32, Ptr{UInt8}, Int32, Ptr{Float32}, Ptr{UInt32}),
        0, 0, K, ntree_limit, nn, feat, cb, sp, lp, x_bin, nobs, nfeats, ft, 0, out, leaf))
    return leaf
end

# ---- evaluation data on the device: replaces CallBack(...) + (cb::CallBack)(logger, iter, tree), src/callback.jl:82-128
# `fit` builds the callback without handing it the cache (src/fit.jl:414), so `init_core` above has to remember the
# cache it created last (e.g. `LAST_CACHE[] = cache`); the reference's `fit` then works unchanged.
const LAST_CACHE = Ref{Union{Nothing,B200Cache}}(nothing)
const METRIC_CODE = Dict(:mse => 0, :rmse => 0, :mae => 1, :logloss => 2, :mlogloss => 3, :gaussian_mle => 4, :gaussian => 4,
    :poisson => 5, :poisson_deviance => 5, :gamma => 6, :gamma_deviance => 6, :tweedie => 7, :tweedie_deviance => 7, :logistic_mle => 8, :quantile => 9, :wmae => 9, :multiquantile => 10)

struct B200CallBack
    feval::Function        # only read by `fit` for is_maximise(cb.feval), src/fit.jl:415
    cache::B200Cache
    metric::Symbol
    initial::Float64
end

metric_value(metric::Symbol, sums) = metric == :rmse ? sqrt(sums[1] / sums[2]) : sums[1] / sums[2]

function EvoTrees.CallBack(params::EvoTypes, m::EvoTree{L,K}, x_eval::AbstractMatrix, y_eval, ::Type{<:GPU};
    w_eval=nothing, offset_eval=nothing) where {L,K}
    cache = LAST_CACHE[]
    x_bin = binarize(x_eval; feature_names=m.info[:feature_names], edges=m.info[:edges])
    y = L == EvoTrees.MLogLoss ? EvoTrees.eval_levelcode(y_eval, m.info[:target_levels]) : Float32.(y_eval)
    w = isnothing(w_eval) ? C_NULL : Float32.(w_eval)
    p0 = C_NULL
    if !isnothing(offset_eval)                     # same link transforms as src/callback.jl:110-118
        off = Float32.(offset_eval)
        L == EvoTrees.LogLoss && (off .= EvoTrees.logit.(off))
        L in (EvoTrees.MLogLoss, EvoTrees.Poisson, EvoTrees.Gamma, EvoTrees.Tweedie) && (off .= log.(off))
        L in (EvoTrees.GaussianMLE, EvoTrees.LogisticMLE) && EvoTrees.unconstrain_mle_scale!(off)
        p0 = Matrix{Float32}(reshape(off, size(x_eval, 1), :)')   # K x nobs
    end
    bias = Float32.(m.trees[end].pred[:, 1])
    sums = zeros(Float64, 2)
    GC.@preserve x_bin y w p0 bias check(ccall((:evb_eval_attach, LIB), Int32,
        (Ptr{Cvoid}, Int64, Ptr{UInt8}, Ptr{Cvoid}, Ptr{Float32}, Ptr{Float32}, Ptr{Float32}, Int32, Ptr{Float64}),
        cache.handle, size(x_eval, 1), x_bin, y, w, p0, bias, METRIC_CODE[params.metric], sums))
    return B200CallBack(EvoTrees.metric_dict[params.metric], cache, params.metric, metric_value(params.metric, sums))
end

function (cb::B200CallBack)(logger, iter, tree)
    if iter == 0
        EvoTrees.update_logger!(logger, iter, cb.initial)
    else
        sums = zeros(Float64, 2)
        check(ccall((:evb_eval_sums, LIB), Int32, (Ptr{Cvoid}, Ptr{Float64}), cb.cache.handle, sums))
        EvoTrees.update_logger!(logger, iter, metric_value(cb.metric, sums))
    end
    return nothing
end

end # module
