// P/Invoke table of libsharpmind_cuda.so.  One declaration per entry point of include/sharpmind_cuda.h, same order.
// Handles (smc_ctx*, smc_weight*, smc_kv*, smc_model*, smc_gguf*, smc_gather*, smc_q8act*) and device pointers travel as
// nint; host pointers keep their element type.
using System.Runtime.InteropServices;

namespace SharpMind.Cuda;

[StructLayout(LayoutKind.Sequential)]
public struct SmcSampling
{
    public float Temperature;
    public int TopK;      // 0 = off
    public float TopP;    // 1 = off
    public float MinP;    // 0 = off
}

/// <summary>Field-for-field mirror of <c>smc_model_desc</c>. Array members point at <c>NLayers</c> entries.</summary>
[StructLayout(LayoutKind.Sequential)]
public unsafe struct SmcModelDesc
{
    public int NLayers, Hidden, NHeads, NKvHeads, HeadDim, Ffn, Vocab, MaxSeq;
    public float Eps, RopeTheta;
    public int Neox, QkNorm;
    public nint* Wq, Wk, Wv, Wo, Wgu, Wdown;          // smc_weight* per layer
    public nint* Norm1, Norm2, QNorm, KNorm;          // device float* per layer
    public nint FinalNorm;                            // device float*
    public nint LmHead;                               // smc_weight*
    public nint* Bq, Bk, Bv, Bo, Bgu, Bdown;          // null, or device float* per layer (entries may be null)
    public int KvDtype;                               // 0 = fp32 cache, 8 = Q8_0 rows
}

internal static unsafe partial class Native
{
    const string Lib = "sharpmind_cuda";   // libsharpmind_cuda.so next to the assembly

    // status codes (sharpmind_cuda.h)
    internal const int Ok = 0, EInvalid = 1, EUnsupported = 2, ESizeMismatch = 3, ECuda = 4, ENotRegistered = 5,
                       ENoDevice = 6, ERange = 7;
    // activation modes
    internal const int ActF32 = 0, ActQ8 = 1, RefOrder = 2;
    // weight registration flags
    internal const int WRepack = 1, WKeepRaw = 2;

    // ---- context
    [LibraryImport(Lib)] internal static partial int smc_version();
    [LibraryImport(Lib)] internal static partial int smc_device_count(out int count);
    [LibraryImport(Lib)] internal static partial int smc_init(int device, out nint ctx);
    [LibraryImport(Lib)] internal static partial void smc_destroy(nint ctx);
    [LibraryImport(Lib)] internal static partial nint smc_last_error(nint ctx);
    [LibraryImport(Lib, StringMarshalling = StringMarshalling.Utf8)]
    internal static partial int smc_set_option(nint ctx, string name, int value);
    [LibraryImport(Lib)] internal static partial int smc_host_register(nint ctx, void* ptr, nuint bytes);
    [LibraryImport(Lib)] internal static partial int smc_host_unregister(nint ctx, void* ptr);
    [LibraryImport(Lib)] internal static partial long smc_raw_tensor_bytes(int dtype, long n, long k);
    [LibraryImport(Lib)] internal static partial int smc_device_status(nint ctx, out int status);
    [LibraryImport(Lib)] internal static partial int smc_synchronize(nint ctx);
    [LibraryImport(Lib)] internal static partial int smc_dev_alloc(nint ctx, nuint bytes, out nint dPtr);
    [LibraryImport(Lib)] internal static partial int smc_dev_free(nint ctx, nint dPtr);
    [LibraryImport(Lib)] internal static partial int smc_copy_to_device(nint ctx, nint dDst, void* hostSrc, nuint bytes, nint stream);
    [LibraryImport(Lib)] internal static partial int smc_copy_to_host(nint ctx, void* hostDst, nint dSrc, nuint bytes, nint stream);

    // ---- weights
    [LibraryImport(Lib)] internal static partial int smc_weight_register(nint ctx, byte* hostRaw, nuint bytes, int dtype,
        int n, int k, int flags, out nint weight);
    [LibraryImport(Lib)] internal static partial int smc_weight_register_dev(nint ctx, nint dRaw, nuint bytes, int dtype,
        int n, int k, int flags, out nint weight);
    [LibraryImport(Lib)] internal static partial int smc_weight_lookup(nint ctx, byte* hostRaw, out nint weight);
    [LibraryImport(Lib)] internal static partial int smc_weight_release(nint ctx, nint weight);
    [LibraryImport(Lib)] internal static partial int smc_weight_shape(nint weight, out int dtype, out int n, out int k);
    [LibraryImport(Lib)] internal static partial int smc_weight_concat_rows(nint ctx, nint* parts, int count, out nint joined);
    [LibraryImport(Lib)] internal static partial int smc_weight_interleave_rows(nint ctx, nint gate, nint up, out nint woven);

    // ---- host-pointer slots (the reference's delegate signatures)
    [LibraryImport(Lib)] internal static partial int smc_qmatmul_host(nint ctx, float* input, byte* hostRaw, float* output,
        int m, int k, int n, int dtype, int mode);
    [LibraryImport(Lib)] internal static partial int smc_qmatmul_host_w(nint ctx, float* input, nint weight, float* output,
        int m, int k, int n, int mode);
    [LibraryImport(Lib)] internal static partial int smc_vecdot_host(nint ctx, float* input, byte* hostRaw, int col, int k,
        int dtype, out float result);
    [LibraryImport(Lib)] internal static partial int smc_swiglu_host(nint ctx, float* gate, float* up, float* dst, int n);
    [LibraryImport(Lib)] internal static partial int smc_silu_host(nint ctx, float* src, float* dst, int n);
    [LibraryImport(Lib)] internal static partial int smc_softmax_row_host(nint ctx, float* src, float* dst, int n);
    [LibraryImport(Lib)] internal static partial int smc_rmsnorm_row_host(nint ctx, float* src, float* weight, float* dst,
        int n, float rmsInv);
    [LibraryImport(Lib)] internal static partial int smc_sdpa_host(nint ctx, float* q, float* k, float* v, float* o,
        int seqLen, int kvLen, int headDim, float scale, int causal, int qStride, int oStride, float alibiSlope);

    // ---- device-resident ops
    [LibraryImport(Lib)] internal static partial int smc_qmatmul_dev(nint ctx, nint dIn, nint weight, nint dOut, int m, int mode, nint stream);
    [LibraryImport(Lib)] internal static partial int smc_add_bias_dev(nint ctx, nint dOut, nint dBias, int rows, int n, nint stream);
    [LibraryImport(Lib)] internal static partial int smc_linear_dev(nint ctx, nint dIn, nint weight, nint dBias, nint dOut, int m, int mode, nint stream);
    [LibraryImport(Lib)] internal static partial int smc_q8act_create(nint ctx, int maxRows, int maxK, out nint act);
    [LibraryImport(Lib)] internal static partial int smc_q8act_destroy(nint ctx, nint act);
    [LibraryImport(Lib)] internal static partial int smc_quantize_q8_dev(nint ctx, nint dX, int m, int k, nint act, nint stream);
    [LibraryImport(Lib)] internal static partial int smc_q8act_read(nint ctx, nint act, sbyte* q, ushort* dBits);
    [LibraryImport(Lib)] internal static partial int smc_qmatmul_tc_dev(nint ctx, nint dIn, nint weight, nint dOut, int m, nint stream);
    [LibraryImport(Lib)] internal static partial int smc_qmatmul_q8_dev(nint ctx, nint act, nint weight, nint dOut, nint stream);
    [LibraryImport(Lib)] internal static partial int smc_qmatmul_q8_noalloc(nint ctx, nint dIn, nint weight, nint dOut, int m, nint stream);
    [LibraryImport(Lib)] internal static partial int smc_block_isums_dev(nint ctx, nint act, int m, nint weight, int col0, int col1, nint dSums, nint stream);
    [LibraryImport(Lib)] internal static partial int smc_quantize_weights_dev(nint ctx, int dtype, nint dValues, long n, nint dRaw, nint stream);
    [LibraryImport(Lib)] internal static partial int smc_rmsnorm_dev(nint ctx, nint dX, nint dW, nint dOut, int rows, int n, float eps, nint stream);
    [LibraryImport(Lib)] internal static partial int smc_swiglu_dev(nint ctx, nint dGate, nint dUp, nint dDst, int rows, int f, int ld, nint stream);
    [LibraryImport(Lib)] internal static partial int smc_silu_dev(nint ctx, nint dSrc, nint dDst, long n, nint stream);
    [LibraryImport(Lib)] internal static partial int smc_softmax_dev(nint ctx, nint dSrc, nint dDst, int rows, int n, nint stream);
    [LibraryImport(Lib)] internal static partial int smc_rope_tables(nint ctx, float theta, int ropeDim, int maxSeq, nint dCos, nint dSin);
    [LibraryImport(Lib)] internal static partial int smc_rope_dev(nint ctx, nint dX, int seq, int heads, int headDim, int ropeDim,
        int posOffset, nint dCos, nint dSin, int neox, nint stream);
    [LibraryImport(Lib)] internal static partial int smc_add_dev(nint ctx, nint dX, nint dY, long n, nint stream);
    [LibraryImport(Lib)] internal static partial int smc_add_rmsnorm_dev(nint ctx, nint dX, nint dY, nint dW, nint dOut, int rows, int n, float eps, nint stream);
    [LibraryImport(Lib)] internal static partial int smc_add_rmsnorm_q8_dev(nint ctx, nint dX, nint dY, nint dW, nint dOut, int rows, int n, float eps, nint act, nint stream);
    [LibraryImport(Lib)] internal static partial int smc_swiglu_quantize_q8_dev(nint ctx, nint dGate, nint dUp, int rows, int f, int ld, nint act, nint stream);
    [LibraryImport(Lib)] internal static partial int smc_argmax_dev(nint ctx, nint dLogits, int rows, int n, nint dOut, nint stream);
    [LibraryImport(Lib)] internal static partial int smc_sample_dev(nint ctx, nint dLogits, int rows, int n, in SmcSampling cfg,
        nint dUniform, nint dWork, nint dTokens, nint stream);
    [LibraryImport(Lib)] internal static partial int smc_repetition_penalty_dev(nint ctx, nint dLogits, int rows, int n, nint dIds,
        int window, float penalty, nint stream);
    [LibraryImport(Lib)] internal static partial int smc_embed_q8_0_dev(nint ctx, nint table, nint dTokens, int count, nint dOut, nint stream);
    [LibraryImport(Lib)] internal static partial int smc_sdpa_decode_dev(nint ctx, nint dQ, nint dK, nint dV, nint dOut, int batch,
        int heads, int kvHeads, int headDim, int kvLen, int maxSeq, float scale, nint stream);
    [LibraryImport(Lib)] internal static partial int smc_kv_append_dev(nint ctx, nint dK, nint dV, nint dKCache, nint dVCache, int batch,
        int kvHeads, int headDim, int pos, int maxSeq, nint stream);
    [LibraryImport(Lib)] internal static partial int smc_qmatmul_swiglu_dev(nint ctx, nint dGate, nint dUp, nint weight, nint dOut, nint stream);
    [LibraryImport(Lib)] internal static partial int smc_qmatmul_swiglu_pairs_dev(nint ctx, nint dX, nint weightInterleaved, nint dAct, nint stream);
    [LibraryImport(Lib)] internal static partial int smc_qmatmul_addnorm_dev(nint ctx, nint dX, nint dAdd, nint dNormW, float eps,
        nint dSum, nint weight, nint dOut, nint stream);

    // ---- KV cache objects (IKVCache)
    [LibraryImport(Lib)] internal static partial int smc_kv_create(nint ctx, int batch, int kvHeads, int maxSeq, int headDim, int kind, out nint kv);
    [LibraryImport(Lib)] internal static partial int smc_kv_destroy(nint ctx, nint kv);
    [LibraryImport(Lib)] internal static partial int smc_kv_length(nint kv);
    [LibraryImport(Lib)] internal static partial int smc_kv_max_seq(nint kv);
    [LibraryImport(Lib)] internal static partial int smc_kv_reset(nint ctx, nint kv);
    [LibraryImport(Lib)] internal static partial int smc_kv_truncate(nint ctx, nint kv, int length);
    [LibraryImport(Lib)] internal static partial int smc_kv_trim_to_last(nint ctx, nint kv, int keep, nint stream);
    [LibraryImport(Lib)] internal static partial int smc_kv_update_dev(nint ctx, nint kv, nint dK, nint dV, int batch, int seqLen, nint stream);
    [LibraryImport(Lib)] internal static partial long smc_kv_snapshot_bytes(nint kv);
    [LibraryImport(Lib)] internal static partial int smc_kv_snapshot(nint ctx, nint kv, void* hostK, void* hostV, long bytesEach, out int position);
    [LibraryImport(Lib)] internal static partial int smc_kv_restore(nint ctx, nint kv, void* hostK, void* hostV, long bytesEach, int position);
    [LibraryImport(Lib)] internal static partial int smc_sdpa_kv_dev(nint ctx, nint kv, nint dQ, nint dOut, int batch, int heads, int seqLen,
        float scale, nint stream);

    // ---- resident decoder
    [LibraryImport(Lib)] internal static partial int smc_model_create(nint ctx, in SmcModelDesc desc, int maxBatch, out nint model);
    [LibraryImport(Lib)] internal static partial int smc_model_destroy(nint ctx, nint model);
    [LibraryImport(Lib)] internal static partial int smc_model_kv(nint ctx, nint model, out nint dK, out nint dV);
    [LibraryImport(Lib)] internal static partial int smc_model_kv_load(nint ctx, nint model, nint dK, nint dV, int batch, int len, nint stream);
    [LibraryImport(Lib)] internal static partial int smc_decode_step(nint ctx, nint model, nint dTokens, int batch, int pos, int mode,
        nint dLogits, nint dArgmax, nint stream);
    [LibraryImport(Lib)] internal static partial int smc_forward_last_logits(nint ctx, nint model, nint dTokens, int seqLen, int seq, int pos,
        int mode, nint dLogits, nint dArgmax, nint stream);
    [LibraryImport(Lib)] internal static partial int smc_forward_logits(nint ctx, nint model, nint dTokens, int seqLen, int seq, int pos,
        int mode, nint dLogits, nint dArgmax, nint dHidden, nint stream);
    [LibraryImport(Lib)] internal static partial int smc_verify_greedy_dev(nint ctx, nint dArgmax, nint dDraft, int heads, nint dAccepted, nint stream);
    [LibraryImport(Lib)] internal static partial int smc_medusa_predict_dev(nint ctx, nint dHidden, nint dHeadW, nint dHeadB, int k, int hidden,
        nint lmHead, nint dWork, nint dTokens, nint stream);

    // ---- GGUF
    [LibraryImport(Lib, StringMarshalling = StringMarshalling.Utf8)]
    internal static partial int smc_gguf_open(nint ctx, string path, out nint gguf);
    [LibraryImport(Lib)] internal static partial int smc_gguf_close(nint ctx, nint gguf);
    [LibraryImport(Lib)] internal static partial int smc_gguf_tensor_count(nint gguf);
    [LibraryImport(Lib, StringMarshalling = StringMarshalling.Utf8)]
    internal static partial int smc_gguf_find(nint gguf, string name);
    [LibraryImport(Lib)] internal static partial int smc_gguf_tensor_info(nint gguf, int index, out nint name, out int dtype, out int nDims,
        long* dims4, out long bytes);
    [LibraryImport(Lib, StringMarshalling = StringMarshalling.Utf8)]
    internal static partial int smc_gguf_meta_int(nint gguf, string key, out long value);
    [LibraryImport(Lib, StringMarshalling = StringMarshalling.Utf8)]
    internal static partial int smc_gguf_meta_float(nint gguf, string key, out double value);
    [LibraryImport(Lib, StringMarshalling = StringMarshalling.Utf8)]
    internal static partial nint smc_gguf_meta_string(nint gguf, string key);
    [LibraryImport(Lib)] internal static partial int smc_gguf_register(nint ctx, nint gguf, int index, int flags, out nint weight);
    [LibraryImport(Lib)] internal static partial int smc_gguf_read_f32(nint ctx, nint gguf, int index, nint dDst, long count);

    // ---- row-split exchange between GPUs
    [LibraryImport(Lib)] internal static partial int smc_gather_create(nint ctx, int rank, int world, nuint capacityFloats, out nint gather);
    [LibraryImport(Lib)] internal static partial int smc_gather_export(nint ctx, nint gather, byte* handle64);
    [LibraryImport(Lib)] internal static partial int smc_gather_connect(nint ctx, nint gather, byte* handlesWorldTimes64);
    [LibraryImport(Lib)] internal static partial int smc_gather_connect_local(nint ctx, nint gather, nint* all);
    [LibraryImport(Lib)] internal static partial int smc_gather_set_wait_ns(nint ctx, nint gather, ulong ns);
    [LibraryImport(Lib)] internal static partial int smc_gather_buffer(nint ctx, nint gather, out nint dBuf);
    [LibraryImport(Lib)] internal static partial int smc_qmatmul_gather_dev(nint ctx, nint gather, nint dIn, nint weightLocal, int m, int mode, nint stream);
    [LibraryImport(Lib)] internal static partial int smc_qmatmul_reduce_dev(nint ctx, nint gather, nint dIn, nint dUp, nint weightLocal, int m, int mode, nint stream);
    [LibraryImport(Lib)] internal static partial int smc_gather_exchange_dev(nint ctx, nint gather, nuint count, nint stream);
    [LibraryImport(Lib)] internal static partial int smc_gather_destroy(nint ctx, nint gather);

    /// <summary>Status code → the exception type the reference's CPU path throws in the same situation.</summary>
    internal static void Check(nint ctx, int rc)
    {
        if (rc == Ok) return;
        string msg = Marshal.PtrToStringUTF8(smc_last_error(ctx)) ?? $"libsharpmind_cuda status {rc}";
        throw rc switch
        {
            ESizeMismatch or ENotRegistered => new InvalidOperationException(msg),   // InferenceLinearLayer.cs:129-134
            ERange                         => new ArgumentOutOfRangeException(null, msg),
            EInvalid                       => new ArgumentException(msg),
            EUnsupported                   => new NotSupportedException(msg),
            ENoDevice                      => new PlatformNotSupportedException(msg),
            _                              => new InvalidOperationException(msg),   // ECuda: message carries the CUDA error
        };
    }
}
