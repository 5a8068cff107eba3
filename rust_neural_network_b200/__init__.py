"""B200-native neural-network framework with the capabilities of rust-nn 2.1.0.

PyTorch is the tensor/autograd layer; every hot op is a hand-written sm_100a CUDA kernel
(tcgen05 + TMEM + TMA) loaded from ``lib/libb200nn_cuda.so``; the host runtime (checkpoint
format, tokenizer, parsers, tiered store, TCP store) is C++ in ``lib/libb200nn_host.so``.

Every public name of the reference's crate root (rust-nn src/lib.rs:83-154) is importable from this
package root, e.g. ``from rust_neural_network_b200 import Linear, Adam, Trainer, BpeTokenizer``.
Submodules load on first use.
"""
import importlib

VERSION = "2.1.0-b200"
__version__ = VERSION

from . import _native  # noqa: F401

_EXPORTS = {
    "activations": "gelu relu sigmoid softmax tanh",
    "blas": "gemm_strassen saxpy scopy sdot sgemm sgemv snrm2 sscal BlasBackend NativeBackend Transpose GEMM_STRASSEN_THRESHOLD",
    "compression": "automl_search CompressedEmbedding CompressionRecipe CompressionStrategy KnowledgeTransfer LayerDropper MixedSparsity "
                   "ProgressiveShrinking SharedWeights SparseMatrix StructuredPruner",
    "data": "format_listings load_csv load_huggingface load_huggingface_auth load_jsonl load_kaggle load_kaggle_auth load_tsv "
            "make_classification make_regression search_huggingface search_kaggle Column Credentials Dataset DatasetBuilder DatasetListing",
    "models.diffusion": "sinusoidal_embedding DenoiseNet NoiseSchedule ScheduleType DDPM",
    "distill": "DistillConfig DistillResult Distiller ProgressiveDistiller",
    "distributed": "average_gradients clip_gradients flatten_gradients recv_message ring_all_reduce_simulated ring_all_reduce_all send_message "
                   "sync_gradients unflatten_gradients DistributedConfig DistributedWorker Message MessageType TcpStore HeartbeatMonitor",
    "error": "RustNnError ShapeMismatch InvalidNdims InvalidInput IndexOutOfBounds EmptyTensor Serialization DataLoad DimensionError InvalidArgument SerializationError IoError DeviceError NumericalError",
    "finetune": "FastTrainConfig FastTrainer LoraAdapter LrSchedule TrainPoint",
    "fused": "fused_linear sparse_topk_route FusedActivation",
    "gpu": "gpu_add gpu_attention gpu_linear gpu_matmul gpu_mul gpu_relu has_gpu GpuBackend",
    "gpu_kernels": "active_backend backend_report detect_backend extract_kernels kernel_matmul kernel_matmul_with_backend kernel_source "
                   "set_backend GpuBackendKind TileConfig AMD_HIP_KERNEL APPLE_MSL_KERNEL NVIDIA_PTX_KERNEL",
    "grpo": "parse_rust_file AdversarialEpisode CoEvolutionStats CoEvolutionTrainer FileNode GrpoConfig GrpoGroup GrpoStats GrpoTrainer "
            "RepoGraph RewardDimension RewardModel RewardScore RewardWeights StructureEdge StructureEdgeType grpo_loss",
    "gui": "full_dashboard launch tensor_heatmap_html ModelDashboard TrainingDashboard",
    "int8": "igemm igemm_scalar Int8Linear Int8Weights",
    "interactive": "run_repl Session process_command",
    "linear_attention": "KernelKind LinearAttentionLayer",
    "models.looped_transformer": "AttentionKind LoopedTransformer MultiHeadAttention Transformer TransformerBlock",
    "models.lm": "LoopedTransformerLM",
    "loss": "BCELoss BCEWithLogitsLoss CrossEntropyLoss HuberLoss L1Loss Loss MSELoss",
    "models.mamba": "HybridMamba Mamba MambaBlock",
    "models.moe": "NormalMoE FineGrainedMoE MoETransformerLM",
    "nn": "attention flash_attention BatchNorm1D Dropout FakeQuantize Flatten LayerNorm Linear Module RNNCell ReLU Recursive Sequential "
          "Sigmoid Softmax Tanh CSA GELU HCA SiLU Embedding",
    "offload": "MemoryTier OffloadConfig OffloadModel SsdTensor TieredStore TieredTensor",
    "optim": "Adam Muon MultiOptimizer Optimizer RMSprop SGD",
    "parallel.ddp": "DistributedAdam DistributedMuon",
    "position": "AlibiBias CARoPE LearnedPE PositionalEncoding RoPE SinusoidalPE",
    "quant": "Rotor RotorQuant",
    "quantize": "QuantFormat QuantizedLinear QuantizedModel QuantizedTensor",      # `quantize` itself: the (callable) submodule
    "models.reasoning": "ChainOfThought MarkovianRSA SwiReasoning TreeOfThoughts",
    "rl": "discounted_returns sample_categorical ActorCritic BanditEnv ChainEnv Dqn Environment Ppo Reinforce ReplayBuffer Transition",
    "self_improve": "Critic SelfImprover",
    "serialize": "deserialize load_model safetensors_export safetensors_import save_model save_model_named",   # `serialize`: callable submodule
    "simd": "simd_add simd_features simd_matmul simd_mul simd_relu simd_scale simd_sum",
    "tensor": "Tensor",
    "ternary": "ternarize TernaryLinear TernaryModel TernaryTensor",
    "tokenizer": "BpeTokenizer MergeScoring",
    "train": "SimpleDataLoader Trainer",
}
_ALIASES = {"blas_matmul": ("blas", "matmul")}        # `pub use blas::matmul as blas_matmul`

_WHERE = {name: (mod, name) for mod, names in _EXPORTS.items() for name in names.split()}
_WHERE.update(_ALIASES)
_SUBMODULES = {"activations", "blas", "compiled", "cpu_ref", "config", "compression", "data", "distill", "distributed", "error", "finetune", "fused", "gpu", "gpu_kernels",
               "grpo", "gui", "int8", "interactive", "linear_attention", "loss", "nn", "offload", "optim", "position", "quant", "quantize", "rl",
               "quantize", "self_improve", "serialize", "simd", "tensor", "ternary", "tokenizer", "train", "models", "ops", "parallel", "utils"}
_MODEL_MODULES = {"looped_transformer", "mamba", "diffusion", "reasoning"}       # crate-root modules that live under models/

__all__ = sorted(set(_WHERE) | _SUBMODULES | _MODEL_MODULES | {"VERSION"})


def __getattr__(name):
    if name in _WHERE:
        mod, attr = _WHERE[name]
        value = getattr(importlib.import_module(f"{__name__}.{mod}"), attr)
        globals()[name] = value
        return value
    if name in _MODEL_MODULES:
        m = importlib.import_module(f"{__name__}.models.{name}")
        globals()[name] = m
        return m
    if name in _SUBMODULES:
        return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def __dir__():
    return __all__
