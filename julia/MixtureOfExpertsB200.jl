# MixtureOfExpertsB200.jl - Julia host side of libmoe_b200.so.
#
# Keeps the names of MixtureOfExperts.jl for the MoE-layer forward path (create_moe_config,
# MoELayer, TopKGating, SwitchGating, SharedExpertGating, GatedExpert, StandardExpert,
# SwitchTransformerLoss, cuda_moe_forward!, create_cuda_moe, to_cuda, to_cpu, and the computing
# part of the Llama2 glue, moe_ffn_forward!) and calls the CUDA kernels through the C ABI of
# include/moe_b200.h with ccall.  It replaces src/cuda of the reference; the CPU types of the reference keep working
# next to it.  NOTE: written against the header, not executed - no Julia runtime was available
# where this library was developed.
module MixtureOfExpertsB200

export MoEConfig, create_moe_config, MoELayer, create_moe_layer, TopKGating, SwitchGating,
       SharedExpertGating, GatedExpert, StandardExpert, SwitchTransformerLoss, GatingMechanism, LoadBalancingLoss,
       cuda_moe_forward!, create_cuda_moe, to_cuda, to_cpu, reset_stats!, load_balance_score, silu,
       set_router_noise!, enable_aux_free!, aux_free_state, moe_ffn_forward!, moe_ffn_forward_batch!, release_device_layers!

const LIB = get(ENV, "MOE_B200_LIB", joinpath(@__DIR__, "..", "mixtureofexperts_b200", "lib", "libmoe_b200.so"))

# ---- enums of moe_b200.h -------------------------------------------------------------------
const GATE_TOPK, GATE_SWITCH, GATE_SHARED_TOPK = Int32(0), Int32(1), Int32(2)
const ACT_SILU, ACT_GELU_TANH, ACT_RELU, ACT_IDENTITY = Int32(0), Int32(1), Int32(2), Int32(3)
const DTYPE_F32, DTYPE_BF16 = Int32(0), Int32(1)
const SHARED_NONE, SHARED_GATING, SHARED_LAYER_BLEND = Int32(0), Int32(1), Int32(2)
const LAYOUT_IN_CONTIG, LAYOUT_OUT_CONTIG = Int32(0), Int32(1)

struct CMoeConfig            # moe_config_t
    num_experts::Int32; num_shared::Int32; top_k::Int32
    input_dim::Int32; hidden_dim::Int32; output_dim::Int32
    gate_kind::Int32; activation::Int32; compute_dtype::Int32; shared_mode::Int32
    balance_alpha::Float32; z_loss_weight::Float32
    index_base::Int32; bias_gates_only::Int32
    capacity_factor::Float32; drop_tokens::Int32; expert_kind::Int32
end

struct CForwardOutputs       # moe_forward_outputs_t (all nullable)
    loss::Ptr{Float32}; indices::Ptr{Int32}; gates::Ptr{Float32}; probs::Ptr{Float32}
    logits::Ptr{Float32}; tokens_per_expert::Ptr{Int64}; routing_entropy::Ptr{Float32}
end

last_error() = unsafe_string(ccall((:moe_last_error, LIB), Cstring, ()))
check(code::Integer) = code == 0 ? nothing : error("moe_b200 [$code]: $(last_error())")

# ---- operator types (same names and fields as the reference) --------------------------------
abstract type GatingMechanism end
abstract type LoadBalancingLoss end

struct TopKGating <: GatingMechanism          # src/gating/topk.jl:16-22
    k::Int
    use_softmax_renorm::Bool
    use_raw_logits::Bool
end
TopKGating(k::Int) = TopKGating(k, true, false)
struct SwitchGating <: GatingMechanism end    # src/gating/switch.jl:7
struct SharedExpertGating <: GatingMechanism  # src/gating/advanced.jl:74-78
    num_shared::Int
    base_gate::GatingMechanism
    num_experts::Int
end
struct SwitchTransformerLoss <: LoadBalancingLoss   # src/balancing/losses.jl:11-13
    α::Float32
end

silu(x) = x * (one(x) / (one(x) + exp(-x)))         # src/experts/gated.jl:36
gelu_tanh(x) = 0.5f0 * x * (1 + tanh(sqrt(2f0 / π) * (x + 0.044715f0 * x^3)))

struct GatedExpert{A}                               # src/experts/gated.jl:6-27
    w1::Matrix{Float32}   # (hidden x input)  Flux Dense.weight layout
    w2::Matrix{Float32}   # (output x hidden)
    w3::Matrix{Float32}   # (hidden x input)
    activation::A
end
function GatedExpert(input_dim::Int, hidden_dim::Int, output_dim::Int, activation)
    σ = sqrt(2.0f0 / input_dim)
    GatedExpert(randn(Float32, hidden_dim, input_dim) .* σ, randn(Float32, output_dim, hidden_dim) .* σ,
                randn(Float32, hidden_dim, input_dim) .* σ, activation)
end

struct StandardExpert{A}                            # src/experts/standard.jl:8-36 (dropout not offered)
    w1::Matrix{Float32}                      # (hidden x input)
    w2::Matrix{Float32}                      # (output x hidden)
    b1::Union{Vector{Float32}, Nothing}
    b2::Union{Vector{Float32}, Nothing}
    activation::A
end
function StandardExpert(input_dim::Int, hidden_dim::Int, output_dim::Int, activation; bias::Bool = true)
    StandardExpert(randn(Float32, hidden_dim, input_dim) .* sqrt(2.0f0 / input_dim),
                   randn(Float32, output_dim, hidden_dim) .* sqrt(2.0f0 / hidden_dim),
                   bias ? zeros(Float32, hidden_dim) : nothing, bias ? zeros(Float32, output_dim) : nothing, activation)
end

Base.@kwdef struct MoEConfig                        # src/core/moe_layer.jl:4-29
    num_experts::Int = 8
    expert_type::Symbol = :standard
    input_dim::Int = 768
    hidden_dim::Int = 3072
    output_dim::Int = 768
    activation::Function = gelu_tanh
    expert_dropout::Float32 = 0.0f0
    gate_type::GatingMechanism = TopKGating(2)
    top_k::Int = 2
    noise_scale::Float32 = 0.0f0
    use_noise_network::Bool = false
    use_fp32_router::Bool = true
    balance_loss::LoadBalancingLoss = SwitchTransformerLoss(0.01f0)
    z_loss_weight::Float32 = 0.001f0
    capacity_factor::Float32 = 1.25f0
    drop_tokens::Bool = false
    use_cur::Bool = false
    cur_rank::Union{Int, Nothing} = nothing
    num_shared_experts::Int = 0
end
create_moe_config(; kwargs...) = MoEConfig(; kwargs...)

# MoEConfig.activation is any callable; the library has four.  Identity first, then a probe.
function activation_enum(f)::Int32
    f === silu && return ACT_SILU
    f === gelu_tanh && return ACT_GELU_TANH
    f === identity && return ACT_IDENTITY
    xs = Float32[-3, -1, -0.25, 0, 0.5, 2]
    got = Float32[f(x) for x in xs]
    for (g, e) in ((silu, ACT_SILU), (gelu_tanh, ACT_GELU_TANH), (x -> max(x, 0f0), ACT_RELU), (identity, ACT_IDENTITY))
        all(isapprox.(got, g.(xs); rtol = 1f-5, atol = 1f-6)) && return e
    end
    error("activation $f is not one of silu/gelu/relu/identity (no CPU fallback exists)")
end

gate_kind(g::TopKGating) = (GATE_TOPK, g.k, 0)
gate_kind(::SwitchGating) = (GATE_SWITCH, 1, 0)
gate_kind(g::SharedExpertGating) = (GATE_SHARED_TOPK, gate_kind(g.base_gate)[2], g.num_shared)

mutable struct MoELayer                              # src/core/moe_layer.jl:34-63
    experts::Vector{Any}                             # GatedExpert or StandardExpert
    router_weight::Matrix{Float32}                   # (E_router x input_dim), Router.weight
    balance_loss::LoadBalancingLoss
    config::MoEConfig
    training_stats::Dict{Symbol, Any}
    handle::Ptr{Cvoid}
end

function MoELayer(config::MoEConfig; device::Int = 0, compute_dtype::Symbol = :f32)
    gated = config.expert_type == :gated          # create_experts: anything else is a StandardExpert
    gated || config.expert_dropout == 0 || error("expert_dropout > 0 is not accelerated")
    kind, k, gate_shared = gate_kind(config.gate_type)
    shared_mode = gate_shared > 0 ? SHARED_GATING : (config.num_shared_experts > 0 ? SHARED_LAYER_BLEND : SHARED_NONE)
    nshared = gate_shared > 0 ? gate_shared : config.num_shared_experts
    c = CMoeConfig(config.num_experts, nshared, k, config.input_dim, config.hidden_dim, config.output_dim,
                   kind, activation_enum(config.activation), compute_dtype == :bf16 ? DTYPE_BF16 : DTYPE_F32,
                   shared_mode, config.balance_loss.α, config.z_loss_weight, 1, 0,
                   config.capacity_factor, config.drop_tokens ? 1 : 0, gated ? 0 : 1)
    h = Ref{Ptr{Cvoid}}(C_NULL)
    check(ccall((:moe_layer_create, LIB), Cint, (Ref{CMoeConfig}, Cint, Ref{Ptr{Cvoid}}), c, device, h))
    experts = [(gated ? GatedExpert : StandardExpert)(config.input_dim, config.hidden_dim, config.output_dim,
                                                      config.activation) for _ in 1:config.num_experts]
    e_router = shared_mode == SHARED_LAYER_BLEND ? config.num_experts - nshared : config.num_experts
    lim = sqrt(6.0f0 / (config.input_dim + e_router))            # Flux Dense default: Glorot uniform
    router = (rand(Float32, e_router, config.input_dim) .* 2 .- 1) .* lim
    stats = Dict{Symbol, Any}(:tokens_per_expert => zeros(Int, config.num_experts),
                              :routing_entropy => Float32[], :capacity_overflow => 0)
    moe = MoELayer(experts, router, config.balance_loss, config, stats, h[])
    finalizer(m -> ccall((:moe_layer_destroy, LIB), Cint, (Ptr{Cvoid},), m.handle), moe)
    sync_weights!(moe)
    return moe
end

"Copy the (possibly modified) Julia-side weights into the device handle."
function sync_weights!(moe::MoELayer)
    for (i, e) in enumerate(moe.experts)
        # Flux (out x in) column-major arrays: the OUT index is contiguous
        if e isa StandardExpert
            check(ccall((:moe_layer_set_expert_standard, LIB), Cint,
                        (Ptr{Cvoid}, Cint, Ptr{Float32}, Ptr{Float32}, Ptr{Float32}, Ptr{Float32}, Cint, Cint, Cint),
                        moe.handle, i - 1, e.w1, something(e.b1, C_NULL), e.w2, something(e.b2, C_NULL),
                        DTYPE_F32, LAYOUT_OUT_CONTIG, 0))
            continue
        end
        check(ccall((:moe_layer_set_expert, LIB), Cint,
                    (Ptr{Cvoid}, Cint, Ptr{Float32}, Ptr{Float32}, Ptr{Float32}, Cint, Cint, Cint),
                    moe.handle, i - 1, e.w1, e.w2, e.w3, DTYPE_F32, LAYOUT_OUT_CONTIG, 0))
    end
    check(ccall((:moe_layer_set_router, LIB), Cint, (Ptr{Cvoid}, Ptr{Float32}, Ptr{Float32}, Cint, Cint),
                moe.handle, moe.router_weight, C_NULL, LAYOUT_OUT_CONTIG, 0))
end

"(moe::MoELayer)(x; training, return_stats) -> (output, balance_loss[, stats])  (src/core/moe_layer.jl:107-128)"
function (moe::MoELayer)(x::AbstractMatrix; training::Bool = false, return_stats::Bool = false)
    cfg = moe.config
    size(x, 1) == cfg.input_dim || error("x must be (input_dim x T)")
    T = size(x, 2)
    xf = Matrix{Float32}(x)                           # column-major (D x T) = T contiguous rows
    out = Matrix{Float32}(undef, cfg.output_dim, T)
    loss = Ref{Float32}(0)
    tpe = zeros(Int64, cfg.num_experts)
    ent = Ref{Float32}(0)
    GC.@preserve xf out tpe begin
        o = CForwardOutputs(Base.unsafe_convert(Ptr{Float32}, loss), C_NULL, C_NULL, C_NULL, C_NULL,
                            pointer(tpe), Base.unsafe_convert(Ptr{Float32}, ent))
        check(ccall((:moe_layer_forward_host, LIB), Cint,
                    (Ptr{Cvoid}, Ptr{Cvoid}, Cint, Int64, Cint, Ptr{Float32}, Ref{CForwardOutputs}),
                    moe.handle, xf, DTYPE_F32, T, training, out, o))
    end
    if cfg.num_shared_experts == 0                    # update_stats! runs in forward_standard only
        moe.training_stats[:tokens_per_expert] .+= tpe
        push!(moe.training_stats[:routing_entropy], ent[])
    end
    return return_stats ? (out, loss[], moe.training_stats) : (out, loss[])
end

"""
cuda_moe_forward!(moe, x; training) on a device array (src/cuda/layer.jl:3-32).  `x` is anything
with `pointer(x)::CuPtr{Float32}` and `size(x) == (input_dim, T)` (a CUDA.jl CuArray); `out` is a
preallocated (output_dim x T) device array; `stream` a CUstream.  No 1024-token cap.
"""
function cuda_moe_forward!(moe::MoELayer, x_ptr::Ptr{Cvoid}, T::Integer, out_ptr::Ptr{Cvoid};
                           training::Bool = false, loss_ptr::Ptr{Cvoid} = C_NULL, stream::Ptr{Cvoid} = C_NULL)
    o = CForwardOutputs(loss_ptr, C_NULL, C_NULL, C_NULL, C_NULL, C_NULL, C_NULL)
    check(ccall((:moe_layer_forward, LIB), Cint,
                (Ptr{Cvoid}, Ptr{Cvoid}, Cint, Int64, Cint, Ptr{Cvoid}, Ref{CForwardOutputs}, Ptr{Cvoid}),
                moe.handle, x_ptr, DTYPE_F32, T, training, out_ptr, o, stream))
end

create_moe_layer(input_dim::Int, hidden_dim::Int, output_dim::Int; kwargs...) =
    MoELayer(MoEConfig(; input_dim, hidden_dim, output_dim, kwargs...))

function reset_stats!(moe::MoELayer)                  # src/core/moe_layer.jl:271-276
    fill!(moe.training_stats[:tokens_per_expert], 0)
    empty!(moe.training_stats[:routing_entropy])
    moe.training_stats[:capacity_overflow] = 0
    nothing
end

function load_balance_score(counts::AbstractVector)   # src/core/utils.jl:40-52
    n, total = length(counts), sum(counts)
    total == 0 && return 1.0f0
    ideal = total / n
    1.0f0 - sqrt(sum((counts .- ideal) .^ 2) / n) / ideal
end

# ---- the remaining names of src/cuda (src/cuda/utils.jl:4-15) ------------------------------------
"create_cuda_moe(; kwargs...): the reference built a CudaMoELayer from CudaMoEConfig keywords; here it is the same MoELayer."
create_cuda_moe(; device::Int = 0, compute_dtype::Symbol = :f32, kwargs...) =
    MoELayer(create_moe_config(; kwargs...); device = device, compute_dtype = compute_dtype)
"to_cuda(x) / to_cpu(x): the layer takes host arrays (moe(x)) or device pointers (cuda_moe_forward!) directly, so these are the identity."
to_cuda(x::AbstractArray) = x
to_cpu(x::AbstractArray) = Array(x)

# ---- training-time branches that live in the handle ---------------------------------------------
"Router noise (src/core/router.jl:32-41): `draws` is a DEVICE pointer to (E_router x T) standard-normal Float32 draws for the next training forward; C_NULL clears it."
set_router_noise!(moe::MoELayer, draws::Ptr{Cvoid}, noise_scale::Real) =
    check(ccall((:moe_layer_set_router_noise, LIB), Cint, (Ptr{Cvoid}, Ptr{Cvoid}, Cfloat), moe.handle, draws, Float32(noise_scale)))

"AuxiliaryFreeLoss.update_bias! on the device (src/balancing/auxiliary_free.jl:36-71): `bias` goes in as the router's logit bias (bias_gates_only must be 1 in the config the handle was created with)."
function enable_aux_free!(moe::MoELayer, bias::Vector{Float32}, bias_momentum::Vector{Float32}; learning_rate::Real = 0.01,
                          momentum::Real = 0.9, update_freq::Int = 1, update_counter::Int = 0)
    check(ccall((:moe_layer_set_router, LIB), Cint, (Ptr{Cvoid}, Ptr{Float32}, Ptr{Float32}, Cint, Cint),
                moe.handle, moe.router_weight, bias, LAYOUT_OUT_CONTIG, 0))
    check(ccall((:moe_layer_set_aux_free, LIB), Cint, (Ptr{Cvoid}, Cint, Cfloat, Cfloat, Cint, Ptr{Float32}, Int64),
                moe.handle, 1, Float32(learning_rate), Float32(momentum), update_freq, bias_momentum, update_counter))
end
"Forward calls of this layer that were served by replaying a captured CUDA graph (small batches on fixed device buffers)."
function graph_replays(moe::MoELayer)
    n = Ref{Int64}(0)
    check(ccall((:moe_layer_graph_replays, LIB), Cint, (Ptr{Cvoid}, Ref{Int64}), moe.handle, n))
    return n[]
end
function aux_free_state(moe::MoELayer)
    n = size(moe.router_weight, 1)
    bias, mom, cnt = zeros(Float32, n), zeros(Float32, n), Ref{Int64}(0)
    check(ccall((:moe_layer_aux_free_state, LIB), Cint, (Ptr{Cvoid}, Ptr{Float32}, Ptr{Float32}, Ref{Int64}),
                moe.handle, bias, mom, cnt))
    return bias, mom, cnt[]
end

# ---- Llama2 glue ------------------------------------------------------------------------------------
# convert_to_moe and sample_moe of the reference (src/llama2/conversion.jl:43-107,
# src/llama2/generation.jl:38-128) build and walk plain Julia structs; they stay as they are.  The
# only code of that path that computes is moe_ffn_forward! (src/llama2/inference.jl:58-121); the two
# functions below replace its routing + expert loop by one library call on the structs convert_to_moe
# made (duck-typed: `layer.moe_experts[e].w1/.w2/.w3`, `layer.moe_router_weight`, `layer.moe_config`;
# `state.xb`, `state.xb2`, `state.selected_experts`, `state.expert_gates`, `state.expert_load_counts`).
# Llama2.jl stores W as (in x out) column-major and applies W'x, i.e. the IN index is contiguous.

const DEVICE_LAYERS = IdDict{Any, Ptr{Cvoid}}()      # converted layer => handle (made on first use)

function device_layer(layer; device::Int = 0, compute_dtype::Symbol = :f32)
    get!(DEVICE_LAYERS, layer) do
        cfg = layer.moe_config
        dim, hidden = size(layer.moe_experts[1].w1)                      # w1 is (dim x hidden_dim)
        kind, k, _ = gate_kind(cfg.gate_type)
        c = CMoeConfig(length(layer.moe_experts), 0, k, dim, hidden, dim, kind, ACT_SILU,
                       compute_dtype == :bf16 ? DTYPE_BF16 : DTYPE_F32, SHARED_NONE, 0.01f0, 0.0f0, 1, 0, 1.25f0, 0, 0)
        h = Ref{Ptr{Cvoid}}(C_NULL)
        check(ccall((:moe_layer_create, LIB), Cint, (Ref{CMoeConfig}, Cint, Ref{Ptr{Cvoid}}), c, device, h))
        for (i, e) in enumerate(layer.moe_experts)
            check(ccall((:moe_layer_set_expert, LIB), Cint,
                        (Ptr{Cvoid}, Cint, Ptr{Float32}, Ptr{Float32}, Ptr{Float32}, Cint, Cint, Cint),
                        h[], i - 1, e.w1, e.w2, e.w3, DTYPE_F32, LAYOUT_IN_CONTIG, 0))
        end
        check(ccall((:moe_layer_set_router, LIB), Cint, (Ptr{Cvoid}, Ptr{Float32}, Ptr{Float32}, Cint, Cint),
                    h[], layer.moe_router_weight, C_NULL, LAYOUT_IN_CONTIG, 0))
        h[]
    end
end

"Free the device handles made by device_layer (call when a converted model is dropped)."
function release_device_layers!()
    for h in values(DEVICE_LAYERS)
        ccall((:moe_layer_destroy, LIB), Cint, (Ptr{Cvoid},), h)
    end
    empty!(DEVICE_LAYERS)
end

"""
moe_ffn_forward!(state, layer, config; rmsnorm! = nothing): the body of the reference's function
for one token.  `rmsnorm!` is Llama2.rmsnorm! (pass it to have `state.xb` computed here like the
reference does; leave it out if `state.xb` already holds the normalised activations).
"""
function moe_ffn_forward!(state, layer, config; rmsnorm! = nothing)
    rmsnorm! === nothing || rmsnorm!(state.xb, state.x, layer.llama_layer.rms_ffn_weight)
    h = device_layer(layer)
    k = length(state.selected_experts)
    idx = zeros(Int32, k)
    GC.@preserve idx begin
        o = CForwardOutputs(C_NULL, pointer(idx), pointer(state.expert_gates), C_NULL, C_NULL, C_NULL, C_NULL)
        check(ccall((:moe_layer_forward_host, LIB), Cint,
                    (Ptr{Cvoid}, Ptr{Cvoid}, Cint, Int64, Cint, Ptr{Float32}, Ref{CForwardOutputs}),
                    h, state.xb, DTYPE_F32, 1, 0, state.xb2, o))
    end
    for j in 1:k
        state.selected_experts[j] = idx[j]
        idx[j] > 0 && (state.expert_load_counts[idx[j]] += 1)
    end
    return nothing
end

"Prefill: the MoE FFN of one layer for all prompt positions at once; X and OUT are (dim x n) Float32 matrices."
function moe_ffn_forward_batch!(OUT::Matrix{Float32}, X::Matrix{Float32}, layer)
    o = CForwardOutputs(C_NULL, C_NULL, C_NULL, C_NULL, C_NULL, C_NULL, C_NULL)
    check(ccall((:moe_layer_forward_host, LIB), Cint,
                (Ptr{Cvoid}, Ptr{Cvoid}, Cint, Int64, Cint, Ptr{Float32}, Ref{CForwardOutputs}),
                device_layer(layer), X, DTYPE_F32, size(X, 2), 0, OUT, o))
    return OUT
end

end # module
