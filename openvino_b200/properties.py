"""Property names, enums and typed property helpers (``ov.properties``).

Reference: src/inference/include/openvino/runtime/properties.hpp (names and value enums) and the Python
mirror src/bindings/python/src/openvino/properties/. A property is addressed by its string name; the helpers
here are callables that return the name when called without arguments and a ``(name, value)`` pair when
called with one, so both ``core.set_property("CPU", {props.enable_profiling: True})`` and
``core.set_property("CPU", props.enable_profiling(True))`` read naturally.
"""
from __future__ import annotations

import enum
from typing import Any


class _Prop(str):
    """A property name that doubles as a ``(name, value)`` maker."""

    def __new__(cls, name: str, mutability: str = "RW"):
        s = super().__new__(cls, name)
        s.mutability = mutability
        return s

    def __call__(self, *value):
        if not value:
            return str(self)
        return (str(self), value[0])


# ------------------------------------------------------------------ enums
class PerformanceMode(enum.Enum):
    LATENCY = "LATENCY"
    THROUGHPUT = "THROUGHPUT"
    CUMULATIVE_THROUGHPUT = "CUMULATIVE_THROUGHPUT"


class ExecutionMode(enum.Enum):
    PERFORMANCE = "PERFORMANCE"
    ACCURACY = "ACCURACY"


class Priority(enum.Enum):
    LOW = "LOW"
    MEDIUM = "MEDIUM"
    HIGH = "HIGH"
    DEFAULT = "MEDIUM"


class SchedulingCoreType(enum.Enum):
    ANY_CORE = "ANY_CORE"
    PCORE_ONLY = "PCORE_ONLY"
    ECORE_ONLY = "ECORE_ONLY"


class CacheMode(enum.Enum):
    OPTIMIZE_SIZE = "OPTIMIZE_SIZE"
    OPTIMIZE_SPEED = "OPTIMIZE_SPEED"


class WorkloadType(enum.Enum):
    DEFAULT = "DEFAULT"
    EFFICIENT = "EFFICIENT"


class Affinity(enum.Enum):
    NONE = "NONE"
    CORE = "CORE"
    NUMA = "NUMA"
    HYBRID_AWARE = "HYBRID_AWARE"


class LogLevel(enum.Enum):
    NO = "LOG_NONE"
    ERR = "LOG_ERROR"
    WARNING = "LOG_WARNING"
    INFO = "LOG_INFO"
    DEBUG = "LOG_DEBUG"
    TRACE = "LOG_TRACE"


class DeviceType(enum.Enum):
    INTEGRATED = "integrated"
    DISCRETE = "discrete"


# ------------------------------------------------------------------ top-level properties
enable_profiling = _Prop("PERF_COUNT")
cache_dir = _Prop("CACHE_DIR")
cache_mode = _Prop("CACHE_MODE")
cache_encryption_callbacks = _Prop("CACHE_ENCRYPTION_CALLBACKS", "WO")
loaded_from_cache = _Prop("LOADED_FROM_CACHE", "RO")
num_streams = _Prop("NUM_STREAMS")
inference_num_threads = _Prop("INFERENCE_NUM_THREADS")
compilation_num_threads = _Prop("COMPILATION_NUM_THREADS")
affinity = _Prop("AFFINITY")
force_tbb_terminate = _Prop("FORCE_TBB_TERMINATE")
enable_mmap = _Prop("ENABLE_MMAP")
auto_batch_timeout = _Prop("AUTO_BATCH_TIMEOUT")
supported_properties = _Prop("SUPPORTED_PROPERTIES", "RO")
available_devices = _Prop("AVAILABLE_DEVICES", "RO")
model_name = _Prop("NETWORK_NAME", "RO")
optimal_number_of_infer_requests = _Prop("OPTIMAL_NUMBER_OF_INFER_REQUESTS", "RO")
range_for_streams = _Prop("RANGE_FOR_STREAMS", "RO")
range_for_async_infer_requests = _Prop("RANGE_FOR_ASYNC_INFER_REQUESTS", "RO")
optimal_batch_size = _Prop("OPTIMAL_BATCH_SIZE", "RO")
max_batch_size = _Prop("MAX_BATCH_SIZE", "RO")
execution_devices = _Prop("EXECUTION_DEVICES", "RO")
weights_path = _Prop("WEIGHTS_PATH")
key_cache_precision = _Prop("KEY_CACHE_PRECISION")
value_cache_precision = _Prop("VALUE_CACHE_PRECISION")
key_cache_group_size = _Prop("KEY_CACHE_GROUP_SIZE")
value_cache_group_size = _Prop("VALUE_CACHE_GROUP_SIZE")


class _Namespace:
    def __init__(self, **kw):
        self.__dict__.update(kw)


hint = _Namespace(
    performance_mode=_Prop("PERFORMANCE_HINT"),
    num_requests=_Prop("PERFORMANCE_HINT_NUM_REQUESTS"),
    inference_precision=_Prop("INFERENCE_PRECISION_HINT"),
    execution_mode=_Prop("EXECUTION_MODE_HINT"),
    model_priority=_Prop("MODEL_PRIORITY"),
    scheduling_core_type=_Prop("SCHEDULING_CORE_TYPE"),
    enable_hyper_threading=_Prop("ENABLE_HYPER_THREADING"),
    enable_cpu_pinning=_Prop("ENABLE_CPU_PINNING"),
    allow_auto_batching=_Prop("ALLOW_AUTO_BATCHING"),
    dynamic_quantization_group_size=_Prop("DYNAMIC_QUANTIZATION_GROUP_SIZE"),
    kv_cache_precision=_Prop("KV_CACHE_PRECISION"),
    model_distribution_policy=_Prop("MODEL_DISTRIBUTION_POLICY"),
    activations_scale_factor=_Prop("ACTIVATIONS_SCALE_FACTOR"),
    model=_Prop("MODEL_PTR"),
    PerformanceMode=PerformanceMode, ExecutionMode=ExecutionMode, Priority=Priority, SchedulingCoreType=SchedulingCoreType,
)

device = _Namespace(
    id=_Prop("DEVICE_ID"),
    priorities=_Prop("MULTI_DEVICE_PRIORITIES"),
    properties=_Prop("DEVICE_PROPERTIES"),
    full_name=_Prop("FULL_DEVICE_NAME", "RO"),
    architecture=_Prop("DEVICE_ARCHITECTURE", "RO"),
    type=_Prop("DEVICE_TYPE", "RO"),
    gops=_Prop("DEVICE_GOPS", "RO"),
    thermal=_Prop("DEVICE_THERMAL", "RO"),
    uuid=_Prop("DEVICE_UUID", "RO"),
    luid=_Prop("DEVICE_LUID", "RO"),
    capabilities=_Prop("OPTIMIZATION_CAPABILITIES", "RO"),
    Type=DeviceType,
)

log = _Namespace(level=_Prop("LOG_LEVEL"), Level=LogLevel)

streams = _Namespace(num=num_streams, AUTO=-1, NUMA=-2)

intel_auto = _Namespace(
    device_bind_buffer=_Prop("DEVICE_BIND_BUFFER"),
    enable_startup_fallback=_Prop("ENABLE_STARTUP_FALLBACK"),
    enable_runtime_fallback=_Prop("ENABLE_RUNTIME_FALLBACK"),
    schedule_policy=_Prop("SCHEDULE_POLICY"),
)

# Device-specific namespaces of the reference: accepted (and stored) by the CPU device and by AUTO; the CUDA device has its own
intel_cpu = _Namespace(
    denormals_optimization=_Prop("CPU_DENORMALS_OPTIMIZATION"),
    sparse_weights_decompression_rate=_Prop("CPU_SPARSE_WEIGHTS_DECOMPRESSION_RATE"),
    tbb_partitioner=_Prop("TBB_PARTITIONER"),
)
intel_gpu = _Namespace(
    device_total_mem_size=_Prop("GPU_DEVICE_TOTAL_MEM_SIZE", "RO"),
    uarch_version=_Prop("GPU_UARCH_VERSION", "RO"),
    execution_units_count=_Prop("GPU_EXECUTION_UNITS_COUNT", "RO"),
    memory_statistics=_Prop("GPU_MEMORY_STATISTICS", "RO"),
    enable_loop_unrolling=_Prop("GPU_ENABLE_LOOP_UNROLLING"),
    disable_winograd_convolution=_Prop("GPU_DISABLE_WINOGRAD_CONVOLUTION"),
    enable_sdpa_optimization=_Prop("GPU_ENABLE_SDPA_OPTIMIZATION"),
    enable_lora_operation=_Prop("GPU_ENABLE_LORA_OPERATION"),
    enable_kernels_reuse=_Prop("GPU_ENABLE_KERNELS_REUSE"),
    hint=_Namespace(
        queue_throttle=_Prop("GPU_QUEUE_THROTTLE"),
        queue_priority=_Prop("GPU_QUEUE_PRIORITY"),
        host_task_priority=_Prop("GPU_HOST_TASK_PRIORITY"),
        available_device_mem=_Prop("AVAILABLE_DEVICE_MEM_SIZE"),
        dynamic_quantization_group_size_max=_Prop("GPU_DYNAMIC_QUANTIZATION_GROUP_SIZE_MAX"),
    ),
)
intel_npu = _Namespace(
    device_alloc_mem_size=_Prop("NPU_DEVICE_ALLOC_MEM_SIZE", "RO"),
    device_total_mem_size=_Prop("NPU_DEVICE_TOTAL_MEM_SIZE", "RO"),
    driver_version=_Prop("NPU_DRIVER_VERSION", "RO"),
    compilation_mode_params=_Prop("NPU_COMPILATION_MODE_PARAMS"),
    turbo=_Prop("NPU_TURBO"),
    tiles=_Prop("NPU_TILES"),
    max_tiles=_Prop("NPU_MAX_TILES"),
    bypass_umd_caching=_Prop("NPU_BYPASS_UMD_CACHING"),
    defer_weights_load=_Prop("NPU_DEFER_WEIGHTS_LOAD"),
    use_npuw=_Prop("NPU_USE_NPUW"),
)

# Properties of the CUDA (B200) device
cuda = _Namespace(
    use_cuda_graphs=_Prop("CUDA_USE_GRAPHS"),
    tensor_parallel_size=_Prop("CUDA_TENSOR_PARALLEL_SIZE"),
    memory_fraction=_Prop("CUDA_MEMORY_FRACTION"),
    weight_layout=_Prop("CUDA_WEIGHT_LAYOUT"),
    # compile a decoder-only LLM graph into the serving program (paged KV cache, ragged batches, CUDA graphs, fused
    # tensor-parallel collectives) instead of the general graph program; the compiled model then hands out the executor
    # that a continuous-batching pipeline drives
    serving_program=_Prop("CUDA_SERVING_PROGRAM"),
)


def value_to_string(v: Any) -> Any:
    """Enum members compare and store as their string value."""
    if isinstance(v, enum.Enum):
        return v.value
    return v


def normalize(config) -> dict:
    """dict / list of pairs / single pair -> {name: plain value}."""
    if config is None:
        return {}
    if isinstance(config, tuple) and len(config) == 2 and isinstance(config[0], str):
        config = [config]
    items = config.items() if isinstance(config, dict) else config
    out = {}
    for k, v in items:
        out[str(k)] = {str(kk): value_to_string(vv) for kk, vv in v.items()} if isinstance(v, dict) else value_to_string(v)
    return out
