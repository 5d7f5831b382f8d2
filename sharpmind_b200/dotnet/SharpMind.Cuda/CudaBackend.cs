// Process-wide context and the weight registry.  The reference's slots receive raw host pointers
// (QuantizedMatMulFn, QuantizationOps.cs:9); the library finds the device copy by that pointer, so a weight array must
// stay at one address for as long as it is registered: it is pinned here for the life of its layer.
using System.Collections.Concurrent;
using System.Runtime.InteropServices;
using SharpMind.Core.Quantization;

namespace SharpMind.Cuda;

public static unsafe class CudaBackend
{
    /// <summary>Activation arithmetic of the matmul slots: 0 fp32 activations (reference semantics, 1e-5·‖w‖·‖x‖),
    /// 1 Q8_0 activations with exact int32 block sums (the fast decode path), 2 the scalar tier's own order (bit-exact).</summary>
    public static int Mode { get; set; } = Native.ActF32;

    /// <summary>Device index the process-wide context is created on. Set before the first use.</summary>
    public static int Device { get; set; }

    public static bool Enabled => CudaSharpMindConfig.HasCuda;

    private static readonly Lazy<nint> _ctx = new(() =>
    {
        int rc = Native.smc_init(Device, out nint ctx);
        if (rc != Native.Ok)
            throw new PlatformNotSupportedException($"libsharpmind_cuda: smc_init({Device}) failed with status {rc}");
        AppDomain.CurrentDomain.ProcessExit += (_, _) => Native.smc_destroy(ctx);
        return ctx;
    }, LazyThreadSafetyMode.ExecutionAndPublication);

    internal static nint Ctx => _ctx.Value;

    private sealed record Registered(GCHandle Pin, nint Weight, int Dtype, int N, int K);

    // keyed by array identity (IEqualityComparer<object?> is contravariant, so it serves byte[] keys)
    private static readonly ConcurrentDictionary<byte[], Registered> _weights = new(ReferenceEqualityComparer.Instance);

    /// <summary>
    /// Uploads a GGUF-layout weight array and pins it. Call from InferenceLinearLayer.SetRawWeight
    /// (InferenceLinearLayer.cs:200-221) after its byte-count check; the library repeats that check and throws
    /// InvalidOperationException on a mismatch, as the layer does.
    /// </summary>
    public static nint Register(byte[] raw, QuantDType dtype, int outFeatures, int inFeatures, bool keepRaw = false)
    {
        ArgumentNullException.ThrowIfNull(raw);
        if (_weights.TryGetValue(raw, out var have)) return have.Weight;
        var pin = GCHandle.Alloc(raw, GCHandleType.Pinned);
        try
        {
            int flags = Native.WRepack | (keepRaw || Mode == Native.RefOrder ? Native.WKeepRaw : 0);
            Native.Check(Ctx, Native.smc_weight_register(Ctx, (byte*)pin.AddrOfPinnedObject(), (nuint)raw.LongLength,
                                                        (int)dtype, outFeatures, inFeatures, flags, out nint w));
            var entry = new Registered(pin, w, (int)dtype, outFeatures, inFeatures);
            if (_weights.TryAdd(raw, entry)) return w;
            Native.smc_weight_release(Ctx, w);      // another thread registered the same array first
            pin.Free();
            return _weights[raw].Weight;
        }
        catch
        {
            if (pin.IsAllocated) pin.Free();
            throw;
        }
    }

    /// <summary>Releases the device copy and unpins the array (InferenceLinearLayer.Dispose).</summary>
    public static void Release(byte[] raw)
    {
        if (!_weights.TryRemove(raw, out var e)) return;
        Native.smc_weight_release(Ctx, e.Weight);
        e.Pin.Free();
    }

    /// <summary>Handle of a registered array, or 0.</summary>
    public static nint Lookup(byte[] raw) => _weights.TryGetValue(raw, out var e) ? e.Weight : 0;

    /// <summary>smc_device_status: 0, or which bounded device wait ran out (1 ring, 2 exchange, 3 prefill pipeline).</summary>
    public static int DeviceStatus()
    {
        Native.Check(Ctx, Native.smc_device_status(Ctx, out int s));
        return s;
    }

    public static void SetOption(string name, int value) => Native.Check(Ctx, Native.smc_set_option(Ctx, name, value));
}
