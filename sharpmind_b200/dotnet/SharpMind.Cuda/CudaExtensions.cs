// MappingBuilder extension selecting this backend, after the pattern of SharpMind.GPU/GpuExtensions.cs:60-101.
using SharpMind.Core;
using SharpMind.Core.Quantization;

namespace SharpMind.Cuda;

public static class CudaExtensions
{
    // CPU hardware suffixes a mapping value may end in (GpuExtensions.HwSuffixes)
    private static readonly string[] HwSuffixes = ["avx512", "avx2", "fma", "sse", "scalar", "gpu"];

    private static readonly string[] VecDotKeys =
    [
        QuantizationKeys.KeyVecDotQ8_0, QuantizationKeys.KeyVecDotQ4K, QuantizationKeys.KeyVecDotQ6K,
    ];

    private static readonly string[] QmmKeys =
    [
        QuantizationKeys.KeyQuantizedMatMulQ8_0, QuantizationKeys.KeyQuantizedMatMulQ4K, QuantizationKeys.KeyQuantizedMatMulQ6K,
    ];

    /// <summary>
    /// Routes the quantized matmul path (and, with <paramref name="nonQuant"/>, SiLU / SwiGLU / softmax / RMSNorm row and
    /// flash attention) to libsharpmind_cuda. Formats other than Q8_0 / Q4_K / Q6_K keep their CPU kernels.
    /// </summary>
    public static MappingBuilder WithCuda(this MappingBuilder builder, bool nonQuant = true, bool vecDot = true, bool matMul = true,
                                          bool attention = false)
    {
        if (!CudaSharpMindConfig.HasCuda)
            throw new PlatformNotSupportedException("WithCuda: libsharpmind_cuda is missing or reports no CUDA device");
        if (nonQuant)
        {
            TryOverrideCuda(builder, SharpMindConfig.KeyPointWise, only: "silu");
            TryOverrideCuda(builder, SharpMindConfig.KeyGate, only: "swiglu");
            builder.Override(SharpMindConfig.KeySoftmax, CudaSharpMindConfig.ValSoftmax);
            builder.Override(SharpMindConfig.KeyRMSNorm, CudaSharpMindConfig.ValRMSNorm);
        }
        if (vecDot)
            foreach (var key in VecDotKeys) TryOverrideCuda(builder, key);
        if (matMul)
        {
            foreach (var key in QmmKeys) TryOverrideCuda(builder, key);
            // `linear` / `logit` take their hardware part from the suffix of mapping["qmatmul_f32"]
            // (LinearLayerFactory.GetCompound, LinearLayerFactory.cs:41-66), which WithGpu leaves alone: without this
            // line the decoder's linear layers keep the CPU kernels whatever the qmatmul_* keys say.
            builder.Override("qmatmul_f32", CudaSharpMindConfig.ValQMatMulF32);
        }
        if (attention)   // per-head host-pointer calls: worth it only for long contexts; the resident decoder is the fast path
            TryOverrideCuda(builder, SharpMindConfig.KeyAttention, flashOnly: true);
        return builder;
    }

    private static void TryOverrideCuda(MappingBuilder builder, string key, string? only = null, bool flashOnly = false)
    {
        if (!builder.TryGetValue(key, out var val) || val is null) return;
        string stripped = val;
        foreach (var sfx in HwSuffixes)
        {
            if (stripped.EndsWith(sfx) && stripped.Length > sfx.Length)
            {
                stripped = stripped[..^sfx.Length];
                break;
            }
        }
        if (only is not null && stripped != only) return;                 // e.g. gelu / geglu stay on the CPU
        if (flashOnly && !stripped.EndsWith("flash")) stripped += "flash"; // mha → mhaflash: only the flash form exists here
        builder.Override(key, stripped + CudaSharpMindConfig.Suffix);
    }
}
