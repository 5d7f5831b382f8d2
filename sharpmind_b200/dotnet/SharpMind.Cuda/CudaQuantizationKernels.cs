// Kernels contributed to the quantized vec-dot / matmul slots and to the `linear` / `logit` slots.
// Signatures are the reference delegates' (VecDotFn, QuantizedMatMulFn: QuantizationOps.cs:8-9); attribute usage follows
// SharpMind.GPU/GPUQuantizationKernels.Q8.cs:13,158,172.  The weight behind `rawWeights` must have been registered
// (CudaBackend.Register); an unknown pointer is uploaded for the call only, which is correct but pays the copy each time.
using JigSawDotNet;
using SharpMind.Core.Quantization;

namespace SharpMind.Cuda;

public static unsafe class CudaQuantizationKernels
{
    private const int Q8_0 = (int)QuantDType.Q8_0, Q4_K = (int)QuantDType.Q4_K, Q6_K = (int)QuantDType.Q6_K;

    private static void MatMul(int dtype, float* input, byte* rawWeights, float* output, int M, int K, int N)
        => Native.Check(CudaBackend.Ctx, Native.smc_qmatmul_host(CudaBackend.Ctx, input, rawWeights, output, M, K, N, dtype, CudaBackend.Mode));

    private static float VecDot(int dtype, float* input, byte* rawWeights, int col, int inFeatures)
    {
        Native.Check(CudaBackend.Ctx, Native.smc_vecdot_host(CudaBackend.Ctx, input, rawWeights, col, inFeatures, dtype, out float r));
        return r;
    }

    // ---- Q8_0
    [PuzzlePeice(QuantizationKeys.KeyVecDotQ8_0, QuantizationKeys.KeyVecDotQ8_0, CudaSharpMindConfig.ValVecDotQ8_0)]
    public static float VecDotQ8_0_Cuda(float* input, byte* rawWeights, int col, int inFeatures)
        => VecDot(Q8_0, input, rawWeights, col, inFeatures);

    [PuzzlePeice(QuantizationKeys.KeyQuantizedMatMulQ8_0, QuantizationKeys.KeyQuantizedMatMulQ8_0, CudaSharpMindConfig.ValQuantizedMatMulQ8_0_Serial)]
    [PuzzlePeice("linear", "linear", CudaSharpMindConfig.ValLinearQ8_0_Serial)]
    [PuzzlePeice("logit", "logit", CudaSharpMindConfig.ValLinearQ8_0_Serial)]
    public static void QuantizedMatMulQ8_0_Serial_Cuda(float* input, byte* rawWeights, float* output, int M, int K, int N)
        => MatMul(Q8_0, input, rawWeights, output, M, K, N);

    [PuzzlePeice(QuantizationKeys.KeyQuantizedMatMulQ8_0, QuantizationKeys.KeyQuantizedMatMulQ8_0, CudaSharpMindConfig.ValQuantizedMatMulQ8_0_Parallel)]
    [PuzzlePeice("linear", "linear", CudaSharpMindConfig.ValLinearQ8_0_Parallel)]
    [PuzzlePeice("logit", "logit", CudaSharpMindConfig.ValLinearQ8_0_Parallel)]
    public static void QuantizedMatMulQ8_0_Parallel_Cuda(float* input, byte* rawWeights, float* output, int M, int K, int N)
        => MatMul(Q8_0, input, rawWeights, output, M, K, N);

    // ---- Q4_K
    [PuzzlePeice(QuantizationKeys.KeyVecDotQ4K, QuantizationKeys.KeyVecDotQ4K, CudaSharpMindConfig.ValVecDotQ4K)]
    public static float VecDotQ4K_Cuda(float* input, byte* rawWeights, int col, int inFeatures)
        => VecDot(Q4_K, input, rawWeights, col, inFeatures);

    [PuzzlePeice(QuantizationKeys.KeyQuantizedMatMulQ4K, QuantizationKeys.KeyQuantizedMatMulQ4K, CudaSharpMindConfig.ValQuantizedMatMulQ4K_Serial)]
    [PuzzlePeice("linear", "linear", CudaSharpMindConfig.ValLinearQ4K_Serial)]
    [PuzzlePeice("logit", "logit", CudaSharpMindConfig.ValLinearQ4K_Serial)]
    public static void QuantizedMatMulQ4K_Serial_Cuda(float* input, byte* rawWeights, float* output, int M, int K, int N)
        => MatMul(Q4_K, input, rawWeights, output, M, K, N);

    [PuzzlePeice(QuantizationKeys.KeyQuantizedMatMulQ4K, QuantizationKeys.KeyQuantizedMatMulQ4K, CudaSharpMindConfig.ValQuantizedMatMulQ4K_Parallel)]
    [PuzzlePeice("linear", "linear", CudaSharpMindConfig.ValLinearQ4K_Parallel)]
    [PuzzlePeice("logit", "logit", CudaSharpMindConfig.ValLinearQ4K_Parallel)]
    public static void QuantizedMatMulQ4K_Parallel_Cuda(float* input, byte* rawWeights, float* output, int M, int K, int N)
        => MatMul(Q4_K, input, rawWeights, output, M, K, N);

    // ---- Q6_K
    [PuzzlePeice(QuantizationKeys.KeyVecDotQ6K, QuantizationKeys.KeyVecDotQ6K, CudaSharpMindConfig.ValVecDotQ6K)]
    public static float VecDotQ6K_Cuda(float* input, byte* rawWeights, int col, int inFeatures)
        => VecDot(Q6_K, input, rawWeights, col, inFeatures);

    [PuzzlePeice(QuantizationKeys.KeyQuantizedMatMulQ6K, QuantizationKeys.KeyQuantizedMatMulQ6K, CudaSharpMindConfig.ValQuantizedMatMulQ6K_Serial)]
    [PuzzlePeice("linear", "linear", CudaSharpMindConfig.ValLinearQ6K_Serial)]
    [PuzzlePeice("logit", "logit", CudaSharpMindConfig.ValLinearQ6K_Serial)]
    public static void QuantizedMatMulQ6K_Serial_Cuda(float* input, byte* rawWeights, float* output, int M, int K, int N)
        => MatMul(Q6_K, input, rawWeights, output, M, K, N);

    [PuzzlePeice(QuantizationKeys.KeyQuantizedMatMulQ6K, QuantizationKeys.KeyQuantizedMatMulQ6K, CudaSharpMindConfig.ValQuantizedMatMulQ6K_Parallel)]
    [PuzzlePeice("linear", "linear", CudaSharpMindConfig.ValLinearQ6K_Parallel)]
    [PuzzlePeice("logit", "logit", CudaSharpMindConfig.ValLinearQ6K_Parallel)]
    public static void QuantizedMatMulQ6K_Parallel_Cuda(float* input, byte* rawWeights, float* output, int M, int K, int N)
        => MatMul(Q6_K, input, rawWeights, output, M, K, N);
}
