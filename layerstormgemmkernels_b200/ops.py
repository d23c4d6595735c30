"""Host-side mirror of the reference's Python operator surface for the GGUF decode path
(csrc/bindings_python.cu of kkontosis/LayerStoRmGemmKernels): same names, argument order,
defaults, checks and error types, implemented over the C ABI of liblsg_b200.so.

torch is used for device memory and the current stream only.  Every operator runs
hand-written sm_100a kernels; nothing here computes on the CPU.
"""
import ctypes

import torch

from . import capi

_lib = capi.lib


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _require(cond, msg):
    # the reference raises through TORCH_CHECK -> RuntimeError
    if not cond:
        raise RuntimeError(msg)


def quantize_q8_1(x):
    """bf16 [M,K] -> uint8 [M, K/32, 36] Q8_1 blocks (d, sum, 32 x int8).

    No Python counterpart in the reference (gguf_quantize_q8_1_cuda is C++ only,
    csrc/sm120/gemm/gguf/gguf_mmvq.cu:124-128); exposed for bit-exactness checks.
    """
    _require(x.is_cuda and x.dtype == torch.bfloat16, "quantize_q8_1: x must be BF16 on CUDA")
    _require(x.dim() == 2 and x.is_contiguous(), "quantize_q8_1: x must be contiguous [M, K]")
    M, K = x.shape
    out = torch.empty((M, K // 32, 36), dtype=torch.uint8, device=x.device)
    capi.check(_lib.lsg_quantize_q8_1(_ptr(x), _ptr(out), M, K, _stream()))
    return out


def _gemm_params(A, B_packed, C, type_i, N, K, out_dtype):
    return capi.GgufMmvqParams(M=A.shape[0], N=int(N), K=int(K), A=A.data_ptr(),
                               B=B_packed.data_ptr(), C=C.data_ptr(), type=int(type_i),
                               out_dtype=out_dtype)


def gguf_mmvq(A, B_packed, type, N, K, out_dtype=torch.bfloat16):
    """GGUF integer mat-vec: bf16 A[M,K] @ decode(B)^T -> [M,N].

    Mirrors gguf_mmvq (csrc/bindings_python.cu:613-643).  out_dtype=torch.float32
    returns the un-rounded accumulator (an extension used by the parity tests).
    """
    _require(A.is_cuda and A.dtype == torch.bfloat16, "gguf_mmvq: A must be BF16 on CUDA")
    _require(A.dim() == 2 and A.is_contiguous(), "gguf_mmvq: A must be contiguous [M, K]")
    _require(A.size(1) == K, "gguf_mmvq: A.size(1) != K")
    _require(B_packed.is_cuda and B_packed.dtype == torch.uint8 and B_packed.is_contiguous(),
             "gguf_mmvq: B_packed must be contiguous uint8 on CUDA")
    _require(out_dtype in (torch.bfloat16, torch.float32), "gguf_mmvq: out_dtype bf16 or f32")
    M = A.size(0)
    C = torch.empty((M, N), dtype=out_dtype, device=A.device)
    ws_bytes = _lib.lsg_gguf_mmvq_workspace_bytes(M, int(K))
    ws = torch.empty((max(ws_bytes, 1),), dtype=torch.uint8, device=A.device)
    p = _gemm_params(A, B_packed, C, type, N, K,
                     capi.DTYPE_F32 if out_dtype == torch.float32 else capi.DTYPE_BF16)
    capi.check(_lib.lsg_gguf_mmvq(ctypes.byref(p), _ptr(ws), ws_bytes, _stream()))
    return C


def gguf_mmvq_batch(A, weights, type, out_dtype=torch.bfloat16):
    """Several projections of the same activations: bf16 A[M,K] against each packed weight
    in `weights` (a sequence of (B_packed, N) with one GGUF type and K), through
    lsg_gguf_mmvq_batch, which runs up to four of them per launch.  Returns the list of
    [M, N] results, equal bit for bit to separate gguf_mmvq calls."""
    _require(A.is_cuda and A.dtype == torch.bfloat16 and A.dim() == 2 and A.is_contiguous(),
             "gguf_mmvq_batch: A must be contiguous BF16 [M, K] on CUDA")
    _require(out_dtype in (torch.bfloat16, torch.float32), "gguf_mmvq_batch: out_dtype bf16 or f32")
    M, K = A.size(0), A.size(1)
    weights = list(weights)
    arr = (capi.GgufMmvqParams * max(len(weights), 1))()
    outs = []
    od = capi.DTYPE_F32 if out_dtype == torch.float32 else capi.DTYPE_BF16
    for i, (B, N) in enumerate(weights):
        _require(B.is_cuda and B.dtype == torch.uint8 and B.is_contiguous(),
                 "gguf_mmvq_batch: B_packed must be contiguous uint8 on CUDA")
        C = torch.empty((M, int(N)), dtype=out_dtype, device=A.device)
        outs.append(C)
        arr[i] = capi.GgufMmvqParams(M=M, N=int(N), K=int(K), A=A.data_ptr(), B=B.data_ptr(),
                                     C=C.data_ptr(), type=int(type), out_dtype=od)
    n = len(weights)
    ws_bytes = _lib.lsg_gguf_mmvq_batch_workspace_bytes(arr, n)
    ws = torch.empty((max(ws_bytes, 1),), dtype=torch.uint8, device=A.device)
    capi.check(_lib.lsg_gguf_mmvq_batch(arr, n, _ptr(ws), ws_bytes, _stream()))
    return outs


def gguf_mmvq_host(A_host, B_packed, type, N, K, out=None, workspace=None):
    """The same mat-vec with the activations and the result in host memory.

    A_host: contiguous bf16 [M, K] CPU tensor (page-locked for an asynchronous call);
    B_packed: packed weight on the device; out: optional bf16 or f32 [M, N] CPU tensor
    (page-locked) to receive the result; workspace: optional uint8 device tensor of at
    least lsg_gguf_mmvq_host_workspace_bytes(M, N, K) bytes.  One C call enqueues the
    copy in, the kernels and the copy out on the current stream and returns without
    waiting: synchronize the stream before reading `out`.  No counterpart in the
    reference, whose operators take device tensors only.
    """
    _require(not A_host.is_cuda and A_host.dtype == torch.bfloat16 and A_host.dim() == 2
             and A_host.is_contiguous(), "gguf_mmvq_host: A must be a contiguous BF16 [M, K] CPU tensor")
    _require(A_host.size(1) == K, "gguf_mmvq_host: A.size(1) != K")
    _require(B_packed.is_cuda and B_packed.dtype == torch.uint8 and B_packed.is_contiguous(),
             "gguf_mmvq_host: B_packed must be contiguous uint8 on CUDA")
    M = A_host.size(0)
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16).pin_memory()
    _require(not out.is_cuda and out.is_contiguous() and tuple(out.shape) == (M, N)
             and out.dtype in (torch.bfloat16, torch.float32),
             "gguf_mmvq_host: out must be a contiguous bf16 or f32 [M, N] CPU tensor")
    need = _lib.lsg_gguf_mmvq_host_workspace_bytes(M, int(N), int(K))
    if workspace is None:
        workspace = torch.empty((max(need, 1),), dtype=torch.uint8, device=B_packed.device)
    _require(workspace.is_cuda and workspace.dtype == torch.uint8 and workspace.numel() >= need,
             "gguf_mmvq_host: workspace too small")
    p = capi.GgufMmvqParams(M=M, N=int(N), K=int(K), A=A_host.data_ptr(), B=B_packed.data_ptr(),
                            C=out.data_ptr(), type=int(type),
                            out_dtype=capi.DTYPE_F32 if out.dtype == torch.float32 else capi.DTYPE_BF16)
    capi.check(_lib.lsg_gguf_mmvq_host(ctypes.byref(p), _ptr(workspace), workspace.numel(), _stream()))
    return out


class HostMmvqBatch:
    """Several projections on host-memory activations and results, enqueued by one C call
    (lsg_gguf_mmvq_host_batch).

    items: sequence of (A_host, B_packed, type, N, K, out_host) with the argument meaning of
    gguf_mmvq_host.  The argument block and the device workspace are built once, here; run()
    enqueues the whole batch on the current stream and returns without waiting.  Items that
    share one A tensor (q, k and v of a hidden state) quantize it once.  The tensors are
    held by the object, and every run() reads the activations' current contents.
    """

    def __init__(self, items, workspace=None):
        items = list(items)
        _require(0 < len(items) <= 64, "HostMmvqBatch: 1..64 projections")
        self._keep = items
        self.outs = []
        arr = (capi.GgufMmvqParams * len(items))()
        dev = items[0][1].device
        for i, (A, B, type, N, K, out) in enumerate(items):
            _require(not A.is_cuda and A.dtype == torch.bfloat16 and A.dim() == 2 and A.is_contiguous()
                     and A.size(1) == K, "HostMmvqBatch: A must be a contiguous BF16 [M, K] CPU tensor")
            _require(B.is_cuda and B.dtype == torch.uint8 and B.is_contiguous() and B.device == dev,
                     "HostMmvqBatch: B_packed must be contiguous uint8 on one CUDA device")
            M = A.size(0)
            if out is None:
                out = torch.empty((M, N), dtype=torch.bfloat16).pin_memory()
            _require(not out.is_cuda and out.is_contiguous() and tuple(out.shape) == (M, N)
                     and out.dtype in (torch.bfloat16, torch.float32),
                     "HostMmvqBatch: out must be a contiguous bf16 or f32 [M, N] CPU tensor")
            self.outs.append(out)
            arr[i] = capi.GgufMmvqParams(
                M=M, N=int(N), K=int(K), A=A.data_ptr(), B=B.data_ptr(), C=out.data_ptr(), type=int(type),
                out_dtype=capi.DTYPE_F32 if out.dtype == torch.float32 else capi.DTYPE_BF16)
        self._arr = arr
        self._n = len(items)
        need = _lib.lsg_gguf_mmvq_host_batch_workspace_bytes(arr, self._n)
        if workspace is None:
            workspace = torch.empty((max(need, 1),), dtype=torch.uint8, device=dev)
        _require(workspace.is_cuda and workspace.dtype == torch.uint8 and workspace.numel() >= need,
                 "HostMmvqBatch: workspace too small")
        self.workspace = workspace
        self._ws = ctypes.c_void_p(workspace.data_ptr())
        self._ws_bytes = workspace.numel()

    def enqueue(self):
        """Enqueues the batch on the current stream (one C call) and returns without waiting;
        usable inside a stream capture, e.g. to record several batches into one graph."""
        capi.check(_lib.lsg_gguf_mmvq_host_batch(self._arr, self._n, self._ws, self._ws_bytes, _stream()))

    _enqueue = enqueue

    def capture(self):
        """Record the batch into a CUDA graph; run() then replays it (one launch from the
        host).  Needs page-locked activations and results: their kernels read and write host
        memory directly, so a replay sees the activations' current contents."""
        self._enqueue()                      # first use outside capture
        torch.cuda.current_stream().synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._enqueue()
        self._graph = g
        return self

    def run(self):
        if getattr(self, "_graph", None) is not None:
            self._graph.replay()
        else:
            self._enqueue()
        return self.outs


def gguf_mmvq_q8_1(xq, B_packed, type, N, K, out_dtype=torch.bfloat16):
    """Same mat-vec on pre-quantized activations (uint8 [M, K/32, 36])."""
    _require(xq.is_cuda and xq.dtype == torch.uint8 and xq.is_contiguous(),
             "gguf_mmvq_q8_1: xq must be contiguous uint8 on CUDA")
    M = xq.size(0)
    C = torch.empty((M, N), dtype=out_dtype, device=xq.device)
    p = capi.GgufMmvqParams(M=M, N=int(N), K=int(K), A=None, B=B_packed.data_ptr(),
                            C=C.data_ptr(), type=int(type),
                            out_dtype=capi.DTYPE_F32 if out_dtype == torch.float32 else capi.DTYPE_BF16)
    capi.check(_lib.lsg_gguf_mmvq_q8_1(ctypes.byref(p), _ptr(xq), _stream()))
    return C


def gguf_dequant_gemm(A, B_packed, type, N, K, out_dtype=torch.bfloat16):
    """Lossless-activation golden: bf16 A @ dequant(B)^T (fp32 accumulate).

    Mirrors launch_gguf_dequant_gemm (csrc/sm120/gemm/gguf/gguf_dequant_gemm.cu:309-325),
    which the reference reaches from Python through gguf_grouped_gemm(strategy=0).
    """
    _require(A.is_cuda and A.dtype == torch.bfloat16 and A.is_contiguous(),
             "gguf_dequant_gemm: A must be contiguous BF16 on CUDA")
    M = A.size(0)
    C = torch.empty((M, N), dtype=out_dtype, device=A.device)
    p = _gemm_params(A, B_packed, C, type, N, K,
                     capi.DTYPE_F32 if out_dtype == torch.float32 else capi.DTYPE_BF16)
    capi.check(_lib.lsg_gguf_dequant_gemm(ctypes.byref(p), _stream()))
    return C


def gguf_dequant(B_packed, type):
    """Packed blocks uint8 [N, row_bytes] -> fp32 [N, K]."""
    t = int(type)
    N = B_packed.size(0)
    nblk = B_packed.size(1) // capi.BLOCK_BYTES[t]
    out = torch.empty((N, nblk * capi.BLOCK_VALUES[t]), dtype=torch.float32, device=B_packed.device)
    capi.check(_lib.lsg_gguf_dequant_blocks(_ptr(B_packed), _ptr(out), t, N * nblk, _stream()))
    return out


# ---------------------------------------------------------------------------
# Activation quantizers
# ---------------------------------------------------------------------------
def dynamic_fp8_quant(input, m_major_scales=False):
    """bf16 [M,K] -> (float8_e4m3fn [M,K], fp32 scales [M,ceil(K/128)] or [ceil(K/128),M]).

    Mirrors dynamic_fp8_quant (csrc/bindings_python.cu:32-61).
    """
    _require(input.is_cuda, "dynamic_fp8_quant: input must be on CUDA")
    _require(input.is_contiguous(), "dynamic_fp8_quant: input must be contiguous")
    _require(input.dim() == 2, "dynamic_fp8_quant: input must be 2D [M, K]")
    _require(input.dtype == torch.bfloat16, "dynamic_fp8_quant: input must be BF16")
    M, K = input.shape
    nb = (K + 127) // 128
    out = torch.empty((M, K), dtype=torch.float8_e4m3fn, device=input.device)
    scales = torch.empty((nb, M) if m_major_scales else (M, nb), dtype=torch.float32,
                         device=input.device)
    p = capi.DynamicFp8QuantParams(num_tokens=M, hidden_size=K, input=input.data_ptr(),
                                   output=out.data_ptr(), scales=scales.data_ptr(),
                                   m_major_scales=1 if m_major_scales else 0)
    capi.check(_lib.lsg_dynamic_fp8_quant(ctypes.byref(p), _stream()))
    return out, scales


def weight_fp8_quant(weight):
    """bf16 [N,K] -> (float8_e4m3fn [N,K], fp32 scales [ceil(N/128), ceil(K/128)]): one scale per
    128 x 128 tile.  Mirrors weight_fp8_quant (csrc/bindings_python.cu:444-471)."""
    _require(weight.is_cuda and weight.dtype == torch.bfloat16, "weight_fp8_quant: weight must be BF16 on CUDA")
    _require(weight.dim() == 2 and weight.is_contiguous(), "weight_fp8_quant: weight must be contiguous [N, K]")
    N, K = weight.shape
    out = torch.empty((N, K), dtype=torch.float8_e4m3fn, device=weight.device)
    scales = torch.empty(((N + 127) // 128, (K + 127) // 128), dtype=torch.float32, device=weight.device)
    capi.check(_lib.lsg_weight_fp8_quant(_ptr(weight), _ptr(out), _ptr(scales), N, K, _stream()))
    return out, scales


def fp8_gemm(A, B, scale_A, scale_B, M, N, K, output_dtype):
    """Block-scaled e4m3 GEMM -> [M,N].  Mirrors fp8_gemm (csrc/bindings_python.cu:475-510)."""
    _require(A.is_cuda and B.is_cuda, "fp8_gemm: A and B must be on CUDA")
    _require(A.is_contiguous() and B.is_contiguous(), "fp8_gemm: must be contiguous")
    code, tdtype = _parse_output_dtype(output_dtype)
    D = torch.empty((M, N), dtype=tdtype, device=A.device)
    ws_bytes = _lib.lsg_fp8_gemm_workspace_bytes(int(M), int(N), int(K))
    ws = torch.empty((max(ws_bytes, 1),), dtype=torch.uint8, device=A.device)
    p = capi.Fp8GemmParams(M=int(M), N=int(N), K=int(K), A=A.data_ptr(), B=B.data_ptr(), D=D.data_ptr(),
                           scale_A=scale_A.data_ptr(), scale_B=scale_B.data_ptr(), output_dtype=code)
    capi.check(_lib.lsg_fp8_gemm(ctypes.byref(p), _ptr(ws), ws_bytes, _stream()))
    return D


def fp8_grouped_gemm(A_base, B_base, D_base, scale_A_base, scale_B_base, expert_offsets, problem_sizes, N, K,
                     output_dtype):
    """Grouped block-scaled e4m3 GEMM into D_base (returned).  Mirrors fp8_grouped_gemm
    (csrc/bindings_python.cu:514-545); routed on the device, no host synchronisation."""
    _require(A_base.is_cuda, "fp8_grouped_gemm: A_base must be on CUDA")
    code, _ = _parse_output_dtype(output_dtype)
    E = expert_offsets.size(0) - 1
    T = A_base.size(0)
    ws_bytes = _lib.lsg_fp8_grouped_gemm_workspace_bytes(T, E, int(N), int(K))
    ws = torch.empty((max(ws_bytes, 1),), dtype=torch.uint8, device=A_base.device)
    p = capi.Fp8GroupedGemmParams(
        num_experts=E, N=int(N), K=int(K), A_base=A_base.data_ptr(), B_base=B_base.data_ptr(),
        D_base=D_base.data_ptr(), scale_A_base=scale_A_base.data_ptr(), scale_B_base=scale_B_base.data_ptr(),
        expert_offsets=expert_offsets.data_ptr(),
        problem_sizes=problem_sizes.data_ptr() if problem_sizes is not None else None,
        output_dtype=code, B_ptrs=None, scale_B_ptrs=None)
    capi.check(_lib.lsg_fp8_grouped_gemm(ctypes.byref(p), T, _ptr(ws), ws_bytes, _stream()))
    return D_base


def _nvfp4_grouped(op, fn, x, up, expert_offsets, input_scales):
    _require(x.is_cuda and x.dtype == torch.bfloat16, f"{op}: input must be BF16 on CUDA")
    _require(x.dim() == 2 and x.is_contiguous(), f"{op}: input must be contiguous [T, K]")
    if up is not None:
        _require(up.is_cuda and up.dtype == torch.bfloat16, f"{op}: up must be BF16 on CUDA")
        _require(up.dim() == 2 and up.is_contiguous(), f"{op}: up must be contiguous [T, K]")
        _require(tuple(up.shape) == tuple(x.shape), f"{op}: gate and up must have the same shape")
    _require(expert_offsets.dim() == 1 and expert_offsets.dtype == torch.int32,
             f"{op}: expert_offsets must be 1D int32")
    T, K = x.shape
    E = expert_offsets.numel() - 1
    _require(K % 64 == 0, f"{op}: K must be divisible by 64 "
             "(K/16 groups must align to the 4-group Sm1xx atom)")
    # As the reference binding: the scale buffer's size depends on the padded row total,
    # which needs the offsets on the host (one D2H copy when they live on the device).
    offs_cpu = expert_offsets.cpu().contiguous()
    _require(int(offs_cpu[E]) == T, f"{op}: expert_offsets must end at total_tokens")
    counts = (offs_cpu[1:] - offs_cpu[:-1]).to(torch.int64)
    padded = ((counts + 127) // 128) * 128
    sf_cpu = torch.zeros(E + 1, dtype=torch.int32)
    sf_cpu[1:] = torch.cumsum(padded, 0).to(torch.int32)
    padded_total = int(sf_cpu[E])
    packed = torch.empty((T, K // 2), dtype=torch.uint8, device=x.device)
    scales = torch.zeros((padded_total * (K // 16),), dtype=torch.uint8, device=x.device)
    offs_dev = expert_offsets.contiguous() if expert_offsets.is_cuda else expert_offsets.to(x.device)
    sf_dev = sf_cpu.to(x.device)
    isc = None
    if input_scales is not None:
        _require(input_scales.is_cuda and input_scales.dtype == torch.float32
                 and input_scales.numel() == E,
                 f"{op}: input_scales must be [num_experts] float32 on CUDA")
        isc = input_scales.contiguous()
    p = capi.Nvfp4GroupedQuantParams(
        input=x.data_ptr(), up=up.data_ptr() if up is not None else None,
        output_packed=packed.data_ptr(), output_scales=scales.data_ptr(),
        expert_offsets=offs_dev.data_ptr(), sf_offsets=sf_dev.data_ptr(), total_tokens=T,
        num_experts=E, K=K, input_scales=isc.data_ptr() if isc is not None else None)
    capi.check(fn(ctypes.byref(p), _stream()))
    return packed, scales, sf_dev


def bf16_to_nvfp4_grouped(input, expert_offsets, input_scales=None):
    """Grouped bf16 -> NVFP4 activation quantization; returns (packed, scales, sf_offsets).

    Mirrors bf16_to_nvfp4_grouped (csrc/bindings_python.cu:287-358).
    """
    return _nvfp4_grouped("bf16_to_nvfp4_grouped", _lib.lsg_bf16_to_nvfp4_grouped, input, None,
                          expert_offsets, input_scales)


def silu_mul_to_nvfp4_grouped(gate, up, expert_offsets, input_scales=None):
    """Fused SwiGLU + grouped NVFP4 quantization; returns (packed, scales, sf_offsets).

    Mirrors silu_mul_to_nvfp4_grouped (csrc/bindings_python.cu:362-440).
    """
    return _nvfp4_grouped("silu_mul_to_nvfp4_grouped", _lib.lsg_silu_mul_to_nvfp4_grouped, gate, up,
                          expert_offsets, input_scales)


# ---------------------------------------------------------------------------
# Grouped (MoE) GEMM
# ---------------------------------------------------------------------------
def gguf_grouped_gemm(A_base, expert_offsets, b_ptrs, type, strategy, N, K, force=0,
                      out_dtype=torch.bfloat16, out=None):
    """One MoE projection over E experts: rows [offsets[e], offsets[e+1]) of A_base times
    decode(weight e)^T.  `b_ptrs` is a CUDA int64 tensor of device pointers.
    strategy: 0 = Dequant, 1 = Int; force: 0 auto, 1 mmvq, 2 mmq, 3 host loop.

    Mirrors gguf_grouped_gemm (csrc/bindings_python.cu:553-604): the output comes from
    torch.empty, so rows of empty or skipped experts are uninitialised.  `out` (not in the
    reference) names a caller-owned contiguous [T, N] tensor to write instead.
    """
    _require(A_base.is_cuda and A_base.dtype == torch.bfloat16,
             "gguf_grouped_gemm: A_base must be BF16 on CUDA")
    _require(A_base.dim() == 2 and A_base.is_contiguous(),
             "gguf_grouped_gemm: A_base must be contiguous [T, K]")
    _require(expert_offsets.is_cuda and expert_offsets.dtype == torch.int32,
             "gguf_grouped_gemm: expert_offsets must be int32 on CUDA")
    _require(b_ptrs.is_cuda and b_ptrs.dtype == torch.int64,
             "gguf_grouped_gemm: b_ptrs must be int64 (device pointers) on CUDA")
    T = A_base.size(0)
    E = b_ptrs.numel()
    _require(expert_offsets.numel() == E + 1,
             "gguf_grouped_gemm: expert_offsets must be [num_experts+1]")
    if out is not None:
        _require(out.is_cuda and out.is_contiguous() and tuple(out.shape) == (T, N)
                 and out.dtype in (torch.bfloat16, torch.float32),
                 "gguf_grouped_gemm: out must be a contiguous bf16 or f32 [T, N] CUDA tensor")
        D, out_dtype = out, out.dtype
    else:
        D = torch.empty((T, N), dtype=out_dtype, device=A_base.device)
    p = capi.GgufGroupedGemmParams(
        type=int(type), strategy=int(strategy), num_experts=E, N=int(N), K=int(K),
        A_base=A_base.data_ptr(), D_base=D.data_ptr(), expert_offsets=expert_offsets.data_ptr(),
        B_ptrs=b_ptrs.data_ptr(),
        out_dtype=capi.DTYPE_F32 if out_dtype == torch.float32 else capi.DTYPE_BF16)
    use_tc = int(strategy) == 1 and int(force) != 3 and E > 0 and (int(force) == 2 or (int(force) == 0 and T // E > 8))
    ws_bytes = (_lib.lsg_gguf_grouped_gemm_workspace_bytes_ex(T, int(K), E, int(N)) if use_tc
                else _lib.lsg_gguf_grouped_gemm_workspace_bytes(T, int(K), E))
    ws = torch.empty((max(ws_bytes, 1),), dtype=torch.uint8, device=A_base.device)
    capi.check(_lib.lsg_gguf_grouped_gemm(ctypes.byref(p), T, _ptr(ws), ws_bytes, int(force), _stream()))
    return D


def gguf_moe_ffn(A_base, expert_offsets, gate_ptrs, up_ptrs, down_ptrs, type, H, I, out_dtype=torch.bfloat16,
                 perm=None, top_k=1):
    """Expert feed-forward block over rows grouped by expert, one call:
    down( silu(gate(x)) * up(x) ) with gate/up packed [I, H] and down packed [H, I] per expert
    (`*_ptrs`: CUDA int64 tensors of device pointers).  The same numbers as three
    gguf_grouped_gemm calls (Int strategy) with the activation computed in fp32 and stored as
    bf16 in between.  An addition to the reference's operator set.

    With `perm` (int32, as moe_permutation returns it) A_base is the UNPERMUTED token matrix
    [num_tokens, H] and row i of the block is token perm[i] // top_k: the permute pass of the
    layer is folded into the call."""
    _require(A_base.is_cuda and A_base.dtype == torch.bfloat16 and A_base.dim() == 2 and A_base.is_contiguous(),
             "gguf_moe_ffn: A_base must be contiguous BF16 [T, H] on CUDA")
    _require(A_base.size(1) == H, "gguf_moe_ffn: A_base.size(1) != H")
    _require(expert_offsets.is_cuda and expert_offsets.dtype == torch.int32,
             "gguf_moe_ffn: expert_offsets must be int32 on CUDA")
    E = gate_ptrs.numel()
    for name, ptrs in (("gate_ptrs", gate_ptrs), ("up_ptrs", up_ptrs), ("down_ptrs", down_ptrs)):
        _require(ptrs.is_cuda and ptrs.dtype == torch.int64 and ptrs.numel() == E,
                 f"gguf_moe_ffn: {name} must be int64 (device pointers) on CUDA, one per expert")
    _require(expert_offsets.numel() == E + 1, "gguf_moe_ffn: expert_offsets must be [num_experts+1]")
    T = A_base.size(0)
    if perm is not None:
        _require(perm.is_cuda and perm.dtype == torch.int32 and perm.dim() == 1 and perm.is_contiguous()
                 and int(top_k) >= 1 and perm.numel() == T * int(top_k),
                 "gguf_moe_ffn: perm must be contiguous int32 [num_tokens * top_k] on CUDA")
        T = perm.numel()
    D = torch.empty((T, H), dtype=out_dtype, device=A_base.device)
    p = capi.GgufMoeFfnParams(
        type=int(type), num_experts=E, H=int(H), I=int(I), A_base=A_base.data_ptr(), D_base=D.data_ptr(),
        expert_offsets=expert_offsets.data_ptr(), gate_ptrs=gate_ptrs.data_ptr(), up_ptrs=up_ptrs.data_ptr(),
        down_ptrs=down_ptrs.data_ptr(),
        out_dtype=capi.DTYPE_F32 if out_dtype == torch.float32 else capi.DTYPE_BF16,
        perm=perm.data_ptr() if perm is not None else None, top_k=int(top_k))
    ws_bytes = _lib.lsg_gguf_moe_ffn_workspace_bytes(T, int(H), int(I), E)
    ws = torch.empty((max(ws_bytes, 1),), dtype=torch.uint8, device=A_base.device)
    capi.check(_lib.lsg_gguf_moe_ffn(ctypes.byref(p), T, _ptr(ws), ws_bytes, _stream()))
    return D


def build_active_expert_list(expert_offsets, cap):
    """int32 [cap]: ascending experts with rows, -1 padded (device-side, no sync)."""
    E = expert_offsets.numel() - 1
    out = torch.empty((cap,), dtype=torch.int32, device=expert_offsets.device)
    capi.check(_lib.lsg_build_active_expert_list(_ptr(expert_offsets), E, cap, _ptr(out), _stream()))
    return out


def build_mmq_tile_map(expert_offsets, tile_m, t_max):
    """(tile_expert, tile_mstart), int32 [t_max] each."""
    E = expert_offsets.numel() - 1
    te = torch.empty((t_max,), dtype=torch.int32, device=expert_offsets.device)
    tm = torch.empty((t_max,), dtype=torch.int32, device=expert_offsets.device)
    capi.check(_lib.lsg_build_mmq_tile_map(_ptr(expert_offsets), E, tile_m, t_max, _ptr(te), _ptr(tm),
                                           _stream()))
    return te, tm


def gguf_mmq(A, B_packed, type, N, K, out_dtype=torch.bfloat16):
    """Prefill GEMM on the tensor cores: bf16 A[M,K] @ decode(B)^T -> [M,N] with the
    integer paths' activation quantization.  The reference reaches its mmq kernels only
    through gguf_grouped_gemm(..., force=2); this direct entry is an addition."""
    _require(A.is_cuda and A.dtype == torch.bfloat16 and A.dim() == 2 and A.is_contiguous(),
             "gguf_mmq: A must be contiguous BF16 [M, K] on CUDA")
    _require(A.size(1) == K, "gguf_mmq: A.size(1) != K")
    M = A.size(0)
    C = torch.empty((M, N), dtype=out_dtype, device=A.device)
    ws_bytes = _lib.lsg_gguf_mmq_workspace_bytes(M, int(N), int(K))
    ws = torch.empty((max(ws_bytes, 1),), dtype=torch.uint8, device=A.device)
    p = _gemm_params(A, B_packed, C, type, N, K,
                     capi.DTYPE_F32 if out_dtype == torch.float32 else capi.DTYPE_BF16)
    capi.check(_lib.lsg_gguf_mmq(ctypes.byref(p), _ptr(ws), ws_bytes, _stream()))
    return C


def gguf_mmq_gather(A, B_slab, type, n_local, K, out_ptrs, ldc, col_offset, out_dtype=torch.bfloat16,
                    multicast_ptr=0):
    """gguf_mmq on a column slab of the weight, every output tile stored into each matrix of
    `out_ptrs` (CUDA int64 tensor of device pointers to [M, ldc] matrices of `out_dtype`, this
    GPU's and its peers') at column offset `col_offset`.  `multicast_ptr`: optional NVLink
    multicast address of those matrices (one store reaches every rank)."""
    _require(A.is_cuda and A.dtype == torch.bfloat16 and A.dim() == 2 and A.is_contiguous(),
             "gguf_mmq_gather: A must be contiguous BF16 [M, K] on CUDA")
    _require(out_ptrs.is_cuda and out_ptrs.dtype == torch.int64, "gguf_mmq_gather: out_ptrs must be int64 on CUDA")
    M = A.size(0)
    ws_bytes = _lib.lsg_gguf_mmq_workspace_bytes(M, int(n_local), int(K))
    ws = torch.empty((max(ws_bytes, 1),), dtype=torch.uint8, device=A.device)
    p = capi.GgufMmvqParams(M=M, N=int(n_local), K=int(K), A=A.data_ptr(), B=B_slab.data_ptr(), C=None,
                            type=int(type),
                            out_dtype=capi.DTYPE_F32 if out_dtype == torch.float32 else capi.DTYPE_BF16)
    capi.check(_lib.lsg_gguf_mmq_gather_mc(ctypes.byref(p), _ptr(out_ptrs), out_ptrs.numel(), int(ldc),
                                           int(col_offset), ctypes.c_void_p(int(multicast_ptr) or None),
                                           _ptr(ws), ws_bytes, _stream()))


def gguf_gemm_bf16(A, B_packed, type, N, K, out_dtype=torch.bfloat16):
    """bf16 A[M,K] @ dequant(B)^T -> [M,N] on the tensor cores with unquantized activations
    (the fast sibling of gguf_dequant_gemm)."""
    _require(A.is_cuda and A.dtype == torch.bfloat16 and A.dim() == 2 and A.is_contiguous(),
             "gguf_gemm_bf16: A must be contiguous BF16 [M, K] on CUDA")
    _require(A.size(1) == K, "gguf_gemm_bf16: A.size(1) != K")
    M = A.size(0)
    C = torch.empty((M, N), dtype=out_dtype, device=A.device)
    ws_bytes = _lib.lsg_gguf_gemm_bf16_workspace_bytes(M, int(N), int(K))
    ws = torch.empty((max(ws_bytes, 1),), dtype=torch.uint8, device=A.device)
    p = _gemm_params(A, B_packed, C, type, N, K,
                     capi.DTYPE_F32 if out_dtype == torch.float32 else capi.DTYPE_BF16)
    capi.check(_lib.lsg_gguf_gemm_bf16(ctypes.byref(p), _ptr(ws), ws_bytes, _stream()))
    return C


def _q4k_legacy(name, x_bf16, weight_q4k_packed):
    # checks of q4k_dequant_gemm / q4k_cutlass_gemm, csrc/bindings_python.cu:647-721
    _require(x_bf16.is_cuda and x_bf16.dtype == torch.bfloat16, "x_bf16 must be BF16 on CUDA")
    _require(x_bf16.dim() == 2 and x_bf16.is_contiguous(), "x_bf16 must be contiguous [M, K]")
    _require(weight_q4k_packed.is_cuda and weight_q4k_packed.dtype == torch.uint8,
             "weight_q4k_packed must be uint8 on CUDA")
    _require(weight_q4k_packed.dim() == 2 and weight_q4k_packed.is_contiguous(),
             "weight_q4k_packed must be contiguous [N, K*9/16]")
    K = x_bf16.size(1)
    N = weight_q4k_packed.size(0)
    _require(K % 256 == 0, f"K must be divisible by 256, got K={K}")
    expected = (K // 256) * 144
    _require(weight_q4k_packed.size(1) == expected,
             f"weight row bytes mismatch: expected {expected}, got {weight_q4k_packed.size(1)}")
    return gguf_gemm_bf16(x_bf16, weight_q4k_packed, capi.Q4_K, N, K)


def q4k_dequant_gemm(x_bf16, weight_q4k_packed):
    """x_bf16 @ dequant(W_q4k).T -> BF16 (csrc/bindings_python.cu:647-682)."""
    return _q4k_legacy("q4k_dequant_gemm", x_bf16, weight_q4k_packed)


def q4k_cutlass_gemm(x_bf16, weight_q4k_packed):
    """x_bf16 @ dequant(W_q4k).T -> BF16, the reference's tensor-core variant
    (csrc/bindings_python.cu:686-721); same kernel as q4k_dequant_gemm here."""
    return _q4k_legacy("q4k_cutlass_gemm", x_bf16, weight_q4k_packed)


# ---------------------------------------------------------------------------
# NVFP4 grouped GEMM
# ---------------------------------------------------------------------------
def _parse_output_dtype(s):
    if s in ("bf16", "bfloat16"):
        return capi.DTYPE_BF16, torch.bfloat16
    if s in ("fp16", "float16"):
        return capi.DTYPE_F16, torch.float16
    raise RuntimeError(f"Unknown output dtype: {s}. Expected 'bf16' or 'fp16'.")


def nvfp4_gemm_preprocess(weight_scales, N, K):
    """fp32 (or fp8) weight scales [N, K/16] -> ue4m3 bytes in the interleaved layout.

    Mirrors nvfp4_gemm_preprocess (csrc/bindings_python.cu:115-145)."""
    _require(weight_scales.is_cuda, "weight_scales must be on CUDA")
    _require(weight_scales.dim() == 2 and weight_scales.is_contiguous(),
             "weight_scales must be contiguous [N, K/16]")
    _require(weight_scales.size(0) == N and weight_scales.size(1) == K // 16,
             "weight_scales shape mismatch")
    src = weight_scales.to(torch.float32).contiguous()
    out = torch.zeros((_lib.lsg_nvfp4_sf_buffer_bytes(int(N), int(K)),), dtype=torch.uint8,
                      device=weight_scales.device)
    capi.check(_lib.lsg_nvfp4_reformat_scales(_ptr(src), _ptr(out), int(N), int(K), _stream()))
    return out


def bf16_to_nvfp4(x):
    """bf16 x[M,K] -> (codes uint8 [M, K/2], ue4m3 scales uint8 [sf_buffer_bytes(M, K)]), the
    single-problem quantizer (launch_bf16_to_nvfp4, csrc/smxx/quant/bf16_to_nvfp4.cu:136-140)."""
    _require(x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.is_contiguous(),
             "bf16_to_nvfp4: x must be contiguous BF16 [M, K] on CUDA")
    M, K = x.shape
    _require(K % 16 == 0, "bf16_to_nvfp4: K must be divisible by 16")
    packed = torch.empty((M, K // 2), dtype=torch.uint8, device=x.device)
    scales = torch.zeros((_lib.lsg_nvfp4_sf_buffer_bytes(M, K),), dtype=torch.uint8, device=x.device)
    capi.check(_lib.lsg_bf16_to_nvfp4(_ptr(x), _ptr(packed), _ptr(scales), M, K, _stream()))
    return packed, scales


def nvfp4_dequant_bf16(weight_packed, weight_scales_e4m3, weight_scale_2):
    """NVFP4 weight [N, K/2] + raw ue4m3 scales [N, K/16] + global scalar -> bf16 [N, K]
    (launch_nvfp4_dequant_bf16, csrc/smxx/quant/nvfp4_dequant_bf16.cu; C API only in the
    reference)."""
    _require(weight_packed.is_cuda and weight_packed.dtype == torch.uint8 and weight_packed.dim() == 2
             and weight_packed.is_contiguous(), "nvfp4_dequant_bf16: weight must be contiguous uint8 [N, K/2] on CUDA")
    N, K = weight_packed.size(0), weight_packed.size(1) * 2
    sc = weight_scales_e4m3.view(torch.uint8)
    _require(sc.is_cuda and sc.is_contiguous() and sc.numel() == N * (K // 16),
             "nvfp4_dequant_bf16: scales must be contiguous [N, K/16] e4m3 bytes on CUDA")
    out = torch.empty((N, K), dtype=torch.bfloat16, device=weight_packed.device)
    capi.check(_lib.lsg_nvfp4_dequant_bf16(_ptr(weight_packed), _ptr(sc), float(weight_scale_2), _ptr(out), N, K,
                                           _stream()))
    return out


def nvfp4_gemm(A, B, scale_A, scale_B, M, N, K, alpha, output_dtype):
    """D[M,N] = alpha * (A x SFA) . (B x SFB)^T on pre-quantized operands.
    Mirrors nvfp4_gemm (csrc/bindings_python.cu:64-110)."""
    _require(A.is_cuda and B.is_cuda, "nvfp4_gemm: A and B must be on CUDA")
    _require(scale_A.is_cuda and scale_B.is_cuda, "nvfp4_gemm: scales must be on CUDA")
    _require(A.is_contiguous() and B.is_contiguous(), "nvfp4_gemm: A and B must be contiguous")
    code, tdtype = _parse_output_dtype(output_dtype)
    D = torch.empty((M, N), dtype=tdtype, device=A.device)
    ws_bytes = _lib.lsg_nvfp4_gemm_workspace_bytes(int(M), int(N), int(K))
    ws = torch.empty((max(ws_bytes, 1),), dtype=torch.uint8, device=A.device)
    p = capi.Nvfp4GemmParams(M=int(M), N=int(N), K=int(K), A=A.data_ptr(), B=B.data_ptr(), D=D.data_ptr(),
                             scale_A=scale_A.data_ptr(), scale_B=scale_B.data_ptr(), alpha=float(alpha),
                             output_dtype=code)
    capi.check(_lib.lsg_nvfp4_gemm(ctypes.byref(p), _ptr(ws), ws_bytes, _stream()))
    return D


def nvfp4_gemm_from_bf16(x_bf16, weight_packed_uint8, weight_scales, weight_scale_global):
    """bf16 activations -> NVFP4 quantization -> GEMM against packed NVFP4 weights -> bf16.
    Mirrors nvfp4_gemm_from_bf16 (csrc/bindings_python.cu:147-244): weight_scales either
    [N, K/16] values or the preprocessed 1-D uint8 buffer of nvfp4_gemm_preprocess."""
    _require(x_bf16.is_cuda and x_bf16.dtype == torch.bfloat16, "x_bf16 must be BF16 on CUDA")
    _require(x_bf16.dim() == 2 and x_bf16.is_contiguous(), "x_bf16 must be contiguous [M, K]")
    _require(weight_packed_uint8.is_cuda and weight_packed_uint8.dtype == torch.uint8,
             "weight_packed_uint8 must be uint8 on CUDA")
    _require(weight_packed_uint8.dim() == 2 and weight_packed_uint8.is_contiguous(),
             "weight_packed_uint8 must be contiguous [N, K/2]")
    _require(weight_scales.is_cuda, "weight_scales must be on CUDA")
    M, K = x_bf16.shape
    N = weight_packed_uint8.size(0)
    _require(weight_packed_uint8.size(1) == K // 2, "weight shape mismatch: expected [N, K/2]")
    _require(K % 32 == 0, f"K must be divisible by 32, got K={K}")
    _require(N % 32 == 0, f"N must be divisible by 32, got N={N}")
    if weight_scales.dtype == torch.uint8 and weight_scales.dim() == 1:
        sfb = weight_scales
    else:
        sfb = nvfp4_gemm_preprocess(weight_scales, N, K)
    codes, sfa = bf16_to_nvfp4(x_bf16)
    return nvfp4_gemm(codes, weight_packed_uint8, sfa, sfb, M, N, K, float(weight_scale_global), "bf16")


def query_sf_buffer_size_b(M, N, K):
    return _lib.lsg_nvfp4_sf_buffer_bytes(int(N), int(K))


def query_sf_buffer_size_a(M, N, K):
    return _lib.lsg_nvfp4_sf_buffer_bytes(int(M), int(K))


def nvfp4_grouped_gemm(A_base, B_base, D_base, scale_A_base, scale_B_base, alphas, expert_offsets,
                       sf_offsets, problem_sizes, N, K, output_dtype):
    """NVFP4 grouped GEMM, in place into D_base; returns D_base.

    Mirrors nvfp4_grouped_gemm (csrc/bindings_python.cu:248-283)."""
    _require(A_base.is_cuda, "nvfp4_grouped_gemm: A_base must be on CUDA")
    code, tdtype = _parse_output_dtype(output_dtype)
    _require(D_base.dtype == tdtype, "nvfp4_grouped_gemm: D_base dtype must match output_dtype")
    E = expert_offsets.size(0) - 1
    T = A_base.size(0)
    # the block-scaled tensor-core route needs a tile map only; unaligned views or odd K take the
    # expanded route and its larger workspace
    aligned = all(t.data_ptr() % 16 == 0 for t in (A_base, B_base, scale_A_base, scale_B_base))
    ws_bytes = _lib.lsg_nvfp4_grouped_gemm_workspace_bytes_ex(T, E, int(N), int(K), 0 if aligned else 1)
    ws = torch.empty((max(ws_bytes, 1),), dtype=torch.uint8, device=A_base.device)
    p = capi.Nvfp4GroupedGemmParams(
        num_experts=E, N=int(N), K=int(K), A_base=A_base.data_ptr(), B_base=B_base.data_ptr(),
        D_base=D_base.data_ptr(), scale_A_base=scale_A_base.data_ptr(),
        scale_B_base=scale_B_base.data_ptr(), alphas=alphas.data_ptr(),
        expert_offsets=expert_offsets.data_ptr(), sf_offsets=sf_offsets.data_ptr(),
        problem_sizes=problem_sizes.data_ptr() if problem_sizes is not None else None,
        output_dtype=code, B_ptrs=None, scale_B_ptrs=None)
    capi.check(_lib.lsg_nvfp4_grouped_gemm(ctypes.byref(p), T, _ptr(ws), ws_bytes, _stream()))
    return D_base


# ---------------------------------------------------------------------------
# MoE routing (additions; the reference takes pre-permuted rows)
# ---------------------------------------------------------------------------
def moe_route(logits, top_k):
    """fp32 logits [T,E] -> (topk_idx int32 [T,k], topk_weights fp32 [T,k])."""
    _require(logits.is_cuda and logits.dtype == torch.float32 and logits.is_contiguous(),
             "moe_route: logits must be contiguous fp32 on CUDA")
    T, E = logits.shape
    idx = torch.empty((T, top_k), dtype=torch.int32, device=logits.device)
    w = torch.empty((T, top_k), dtype=torch.float32, device=logits.device)
    capi.check(_lib.lsg_moe_route(_ptr(logits), T, E, int(top_k), _ptr(idx), _ptr(w), _stream()))
    return idx, w


def moe_permutation(topk_idx, num_experts):
    """-> (expert_offsets int32 [E+1], perm int32 [T*k], inv_perm int32 [T*k])."""
    T, k = topk_idx.shape
    dev = topk_idx.device
    offs = torch.empty((num_experts + 1,), dtype=torch.int32, device=dev)
    perm = torch.empty((T * k,), dtype=torch.int32, device=dev)
    inv = torch.empty((T * k,), dtype=torch.int32, device=dev)
    n_scratch = _lib.lsg_moe_permutation_scratch_ints(T, k, int(num_experts))
    scratch = torch.empty((max(int(n_scratch), 1),), dtype=torch.int32, device=dev)
    capi.check(_lib.lsg_moe_permutation(_ptr(topk_idx), T, k, int(num_experts), _ptr(offs), _ptr(perm),
                                        _ptr(inv), _ptr(scratch), _stream()))
    return offs, perm, inv


def ep_expert_order(recv_counts, world, experts_per_rank, rows):
    """recv_counts int32 [world, per] on CUDA -> (local_offsets int32 [per+1], order int32 [rows],
    inv_order int32 [rows]): regrouping of rows received by (source, expert) into (expert, source)."""
    dev = recv_counts.device
    c = recv_counts.to(torch.int32).contiguous()
    offs = torch.empty((experts_per_rank + 1,), dtype=torch.int32, device=dev)
    order = torch.empty((max(rows, 1),), dtype=torch.int32, device=dev)
    inv = torch.empty((max(rows, 1),), dtype=torch.int32, device=dev)
    scratch = torch.empty((2 * world * experts_per_rank,), dtype=torch.int32, device=dev)
    capi.check(_lib.lsg_ep_expert_order(_ptr(c), int(world), int(experts_per_rank), int(rows), _ptr(offs),
                                        _ptr(order), _ptr(inv), _ptr(scratch), _stream()))
    return offs, order[:rows], inv[:rows]


def moe_permute(hidden, perm, top_k):
    rows, H = perm.numel(), hidden.size(1)
    out = torch.empty((rows, H), dtype=torch.bfloat16, device=hidden.device)
    capi.check(_lib.lsg_moe_permute(_ptr(hidden), _ptr(perm), rows, int(top_k), H, _ptr(out), _stream()))
    return out


def moe_unpermute(y, inv_perm, topk_weights):
    T, k = topk_weights.shape
    H = y.size(1)
    out = torch.empty((T, H), dtype=torch.bfloat16, device=y.device)
    capi.check(_lib.lsg_moe_unpermute(_ptr(y), _ptr(inv_perm), _ptr(topk_weights), T, k, H, _ptr(out),
                                      _stream()))
    return out
