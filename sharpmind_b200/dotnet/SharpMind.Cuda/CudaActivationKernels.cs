// Kernels contributed to the activation / norm / attention slots.  Signatures are those of
// SharpMind.GPU/GPUActivationKernels.cs:67-171 (SiLUGPU, SwiGLUGPU, SoftmaxRowGPU, RMSNormRowGPU) and of
// AttentionLayer.ScaledDotProduct (AttentionLayer.cs:258).
using JigSawDotNet;
using SharpMind.Core;

namespace SharpMind.Cuda;

public static unsafe class CudaActivationKernels
{
    [PuzzlePeice(SharpMindConfig.KeyPointWise, SharpMindConfig.KeyPointWise, CudaSharpMindConfig.ValSiLU)]
    public static void SiLUCuda(ReadOnlySpan<float> src, Span<float> dst)
    {
        if (dst.Length < src.Length) throw new ArgumentException("dst is shorter than src");
        fixed (float* s = src, d = dst)
            Native.Check(CudaBackend.Ctx, Native.smc_silu_host(CudaBackend.Ctx, s, d, src.Length));
    }

    [PuzzlePeice(SharpMindConfig.KeyGate, SharpMindConfig.KeyGate, CudaSharpMindConfig.ValSwiGLU)]
    public static void SwiGLUCuda(ReadOnlySpan<float> gate, ReadOnlySpan<float> up, Span<float> dst)
    {
        if (gate.Length != up.Length || dst.Length < gate.Length) throw new ArgumentException("gate / up / dst lengths differ");
        fixed (float* g = gate, u = up, d = dst)
            Native.Check(CudaBackend.Ctx, Native.smc_swiglu_host(CudaBackend.Ctx, g, u, d, gate.Length));
    }

    [PuzzlePeice(SharpMindConfig.KeySoftmax, SharpMindConfig.KeySoftmax, CudaSharpMindConfig.ValSoftmax)]
    public static void SoftmaxRowCuda(ReadOnlySpan<float> src, Span<float> dst)
    {
        if (dst.Length < src.Length) throw new ArgumentException("dst is shorter than src");
        fixed (float* s = src, d = dst)
            Native.Check(CudaBackend.Ctx, Native.smc_softmax_row_host(CudaBackend.Ctx, s, d, src.Length));
    }

    [PuzzlePeice(SharpMindConfig.KeyRMSNorm, SharpMindConfig.KeyRMSNorm, CudaSharpMindConfig.ValRMSNorm)]
    public static void RMSNormRowCuda(ReadOnlySpan<float> src, ReadOnlySpan<float> weight, Span<float> dst, float rmsInv)
    {
        if (weight.Length < src.Length || dst.Length < src.Length) throw new ArgumentException("weight / dst shorter than src");
        fixed (float* s = src, w = weight, d = dst)
            Native.Check(CudaBackend.Ctx, Native.smc_rmsnorm_row_host(CudaBackend.Ctx, s, w, d, src.Length, rmsInv));
    }

    // One kernel serves the three head layouts: the slot is called per (batch, head) with that head's pointers.
    [PuzzlePeice(SharpMindConfig.KeyAttention, SharpMindConfig.KeyAttention, CudaSharpMindConfig.ValMhaFlash)]
    [PuzzlePeice(SharpMindConfig.KeyAttention, SharpMindConfig.KeyAttention, CudaSharpMindConfig.ValGqaFlash)]
    [PuzzlePeice(SharpMindConfig.KeyAttention, SharpMindConfig.KeyAttention, CudaSharpMindConfig.ValMqaFlash)]
    public static void ScaledDotProductFlashCuda(float* q, float* k, float* v, float* o, int seqLen, int kvLen, int headDim,
        float scale, bool causal, int qStride, int oStride, float alibiSlope)
        => Native.Check(CudaBackend.Ctx, Native.smc_sdpa_host(CudaBackend.Ctx, q, k, v, o, seqLen, kvLen, headDim, scale,
                                                             causal ? 1 : 0, qStride, oStride, alibiSlope));
}
