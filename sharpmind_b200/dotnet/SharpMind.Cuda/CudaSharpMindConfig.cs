// Mapping values this backend contributes, named after the pattern of SharpMind.GPU/GPUSharpMindConfig.cs ("…gpu" → "…cuda").
using SharpMind.Core;

namespace SharpMind.Cuda;

public static class CudaSharpMindConfig
{
    public const string Suffix = "cuda";

    public const string ValSiLU = "silucuda";
    public const string ValSwiGLU = "swiglucuda";
    public const string ValSoftmax = "softmaxcuda";
    public const string ValRMSNorm = "rmsnormcuda";

    public const string ValVecDotQ8_0 = "q8_0_cuda";
    public const string ValVecDotQ4K = "q4k_cuda";
    public const string ValVecDotQ6K = "q6k_cuda";

    public const string ValQuantizedMatMulQ8_0_Serial = "qmatmul_q8_0_serial_cuda";
    public const string ValQuantizedMatMulQ4K_Serial = "qmatmul_q4k_serial_cuda";
    public const string ValQuantizedMatMulQ6K_Serial = "qmatmul_q6k_serial_cuda";
    public const string ValQuantizedMatMulQ8_0_Parallel = "qmatmul_q8_0_parallel_cuda";
    public const string ValQuantizedMatMulQ4K_Parallel = "qmatmul_q4k_parallel_cuda";
    public const string ValQuantizedMatMulQ6K_Parallel = "qmatmul_q6k_parallel_cuda";

    // `linear` / `logit` compound names: "<dtype>_<serial|parallel>_<hw>" (LinearLayerFactory.GetCompound,
    // LinearLayerFactory.cs:41-66; the hw part is the suffix of mapping["qmatmul_f32"])
    public const string ValLinearQ8_0_Serial = "q8_0_serial_cuda";
    public const string ValLinearQ8_0_Parallel = "q8_0_parallel_cuda";
    public const string ValLinearQ4K_Serial = "q4k_serial_cuda";
    public const string ValLinearQ4K_Parallel = "q4k_parallel_cuda";
    public const string ValLinearQ6K_Serial = "q6k_serial_cuda";
    public const string ValLinearQ6K_Parallel = "q6k_parallel_cuda";
    public const string ValQMatMulF32 = "qmatmul_f32_parallel_cuda";

    public const string ValMhaFlash = "mhaflashcuda";
    public const string ValGqaFlash = "gqaflashcuda";
    public const string ValMqaFlash = "mqaflashcuda";

    /// <summary>True when the native library loads and reports at least one CUDA device.</summary>
    public static bool HasCuda => _has.Value;

    private static readonly Lazy<bool> _has = new(() =>
    {
        try { return Native.smc_device_count(out int n) == Native.Ok && n > 0; }
        catch (DllNotFoundException) { return false; }
        catch (EntryPointNotFoundException) { return false; }
    }, LazyThreadSafetyMode.ExecutionAndPublication);
}
