// IKVCache (SharpMind.Model/IKVCache.cs) over a device cache object: fp32 rows (KVCache) or Q8_0 rows (QuantizedKVCache).
// Keys and values never visit the host, so the pointer accessors of the interface cannot be served: attention over this
// cache is smc_sdpa_kv_dev (Attend below), which AttentionLayer.Forward calls instead of its per-head loop when the
// cache is a CudaKVCache.
using SharpMind.Core.Tensors;
using SharpMind.Model;

namespace SharpMind.Cuda;

public sealed unsafe class CudaKVCache : IKVCache
{
    public const int KindF32 = 0, KindQ8_0 = 8;

    private nint _kv;
    private readonly int _batch, _kvHeads, _headDim, _kind;
    private DeviceBuffer<float>? _stageK, _stageV;

    public CudaKVCache(int batchSize, int numKvHeads, int maxSeqLen, int headDim, int kind = KindF32)
    {
        (_batch, _kvHeads, _headDim, _kind) = (batchSize, numKvHeads, headDim, kind);
        Native.Check(CudaBackend.Ctx, Native.smc_kv_create(CudaBackend.Ctx, batchSize, numKvHeads, maxSeqLen, headDim, kind, out _kv));
    }

    internal nint Handle => _kv;
    public int Length => Native.smc_kv_length(_kv);
    public int MaxSeqLen => Native.smc_kv_max_seq(_kv);
    public bool IsFull => Length >= MaxSeqLen;
    public bool IsContiguous => false;   // no host-addressable rows

    /// <summary>Appends k, v [batch, seqLen, kvHeads*headDim] held on the host (KVCache.Update).</summary>
    public void Update(Tensor<float> k, Tensor<float> v, int numKvHeads, int headDim)
    {
        if (numKvHeads != _kvHeads || headDim != _headDim) throw new ArgumentException("head layout differs from the cache's");
        int batch = k.Shape[0], seqLen = k.Shape[1];
        long n = (long)batch * seqLen * numKvHeads * headDim;
        if (_stageK is null || _stageK.Length < n)
        {
            _stageK?.Dispose(); _stageV?.Dispose();
            _stageK = new DeviceBuffer<float>(n); _stageV = new DeviceBuffer<float>(n);
        }
        _stageK.Upload(k.Data[..(int)n]);
        _stageV!.Upload(v.Data[..(int)n]);
        UpdateDevice(_stageK.Pointer, _stageV.Pointer, batch, seqLen);
    }

    /// <summary>Appends rows that already live on the device: dK, dV are [batch, seqLen, kvHeads, headDim] fp32.</summary>
    public void UpdateDevice(nint dK, nint dV, int batch, int seqLen)
    {
        int rc = Native.smc_kv_update_dev(CudaBackend.Ctx, _kv, dK, dV, batch, seqLen, 0);
        if (rc == Native.ERange)   // the reference throws InvalidOperationException on overflow (KVCache.cs:89-91)
            throw new InvalidOperationException($"KVCache overflow: position {Length} + seqLen {seqLen} exceeds capacity {MaxSeqLen}.");
        Native.Check(CudaBackend.Ctx, rc);
    }

    /// <summary>Causal attention of the last seqLen positions against the cache; dQ, dOut are [batch, seqLen, heads, headDim].</summary>
    public void Attend(nint dQ, nint dOut, int batch, int heads, int seqLen, float scale)
        => Native.Check(CudaBackend.Ctx, Native.smc_sdpa_kv_dev(CudaBackend.Ctx, _kv, dQ, dOut, batch, heads, seqLen, scale, 0));

    public void Reset() => Native.Check(CudaBackend.Ctx, Native.smc_kv_reset(CudaBackend.Ctx, _kv));

    public void Truncate(int length) => Native.Check(CudaBackend.Ctx, Native.smc_kv_truncate(CudaBackend.Ctx, _kv, length));

    public void TrimToLast(int keep)
    {
        ArgumentOutOfRangeException.ThrowIfNegative(keep);
        Native.Check(CudaBackend.Ctx, Native.smc_kv_trim_to_last(CudaBackend.Ctx, _kv, keep, 0));
    }

    public float* GetKeyPtr(int batchIdx, int position, int kvHead)
        => throw new NotSupportedException("CudaKVCache rows live on the device; use Attend()");

    public float* GetValuePtr(int batchIdx, int position, int kvHead)
        => throw new NotSupportedException("CudaKVCache rows live on the device; use Attend()");

    /// <summary>(position, keys, values) with the active rows of every (sequence, head) packed densely; floats for an
    /// fp32 cache (IKVCache.SnapshotBytes tag 1), Q8_0 blocks of 34 bytes for a Q8_0 cache (tag 3).</summary>
    public object? Snapshot()
    {
        if (Length == 0) return null;
        long bytes = Native.smc_kv_snapshot_bytes(_kv);
        if (_kind == KindF32)
        {
            var k = new float[bytes / sizeof(float)];
            var v = new float[bytes / sizeof(float)];
            int pos;
            fixed (float* pk = k, pv = v)
                Native.Check(CudaBackend.Ctx, Native.smc_kv_snapshot(CudaBackend.Ctx, _kv, pk, pv, bytes, out pos));
            return (pos, k, v);
        }
        else
        {
            var k = new byte[bytes];
            var v = new byte[bytes];
            int pos;
            fixed (byte* pk = k, pv = v)
                Native.Check(CudaBackend.Ctx, Native.smc_kv_snapshot(CudaBackend.Ctx, _kv, pk, pv, bytes, out pos));
            return (pos, k, v);
        }
    }

    public void Restore(object? snapshot)
    {
        switch (snapshot)
        {
            case null:
                return;
            case (int pos, float[] k, float[] v):
                fixed (float* pk = k, pv = v)
                    Native.Check(CudaBackend.Ctx, Native.smc_kv_restore(CudaBackend.Ctx, _kv, pk, pv, (long)k.Length * sizeof(float), pos));
                return;
            case (int pos, byte[] k, byte[] v):
                fixed (byte* pk = k, pv = v)
                    Native.Check(CudaBackend.Ctx, Native.smc_kv_restore(CudaBackend.Ctx, _kv, pk, pv, k.LongLength, pos));
                return;
            default:
                throw new InvalidOperationException($"Unknown KVCache snapshot type: {snapshot.GetType()}");
        }
    }

    public void Dispose()
    {
        if (_kv != 0) { Native.smc_kv_destroy(CudaBackend.Ctx, _kv); _kv = 0; }
        _stageK?.Dispose(); _stageV?.Dispose();
    }
}
