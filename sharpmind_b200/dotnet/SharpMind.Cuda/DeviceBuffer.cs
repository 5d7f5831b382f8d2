// A device allocation owned by managed code (what ILGPU's MemoryBuffer1D is to SharpMind.GPU).
namespace SharpMind.Cuda;

public sealed unsafe class DeviceBuffer<T> : IDisposable where T : unmanaged
{
    public nint Pointer { get; private set; }
    public long Length { get; }

    public DeviceBuffer(long length)
    {
        ArgumentOutOfRangeException.ThrowIfNegativeOrZero(length);
        Length = length;
        Native.Check(CudaBackend.Ctx, Native.smc_dev_alloc(CudaBackend.Ctx, (nuint)(length * sizeof(T)), out nint p));
        Pointer = p;
    }

    public DeviceBuffer(ReadOnlySpan<T> host) : this(host.Length) => Upload(host);

    public void Upload(ReadOnlySpan<T> host, long dstOffset = 0)
    {
        if (dstOffset < 0 || dstOffset + host.Length > Length) throw new ArgumentOutOfRangeException(nameof(host));
        fixed (T* p = host)
            Native.Check(CudaBackend.Ctx, Native.smc_copy_to_device(CudaBackend.Ctx, Pointer + (nint)(dstOffset * sizeof(T)), p,
                                                                   (nuint)((long)host.Length * sizeof(T)), 0));
    }

    public void Download(Span<T> host, long srcOffset = 0)
    {
        if (srcOffset < 0 || srcOffset + host.Length > Length) throw new ArgumentOutOfRangeException(nameof(host));
        fixed (T* p = host)
            Native.Check(CudaBackend.Ctx, Native.smc_copy_to_host(CudaBackend.Ctx, p, Pointer + (nint)(srcOffset * sizeof(T)),
                                                                 (nuint)((long)host.Length * sizeof(T)), 0));
    }

    public void Dispose()
    {
        if (Pointer == 0) return;
        Native.smc_dev_free(CudaBackend.Ctx, Pointer);
        Pointer = 0;
    }
}
