// The resident decoder: Transformer.ForwardLastLogits / Forward (SharpMind.Model/Transformer.cs:417-463) for a
// Llama/Qwen-shaped model whose weights, KV cache and activations stay on the device.  A generator calls Prefill once,
// then Step per token and reads back 4 bytes per sequence (or samples on the device); Medusa / speculative generators
// call ForwardAll + VerifyGreedy and roll back by passing a smaller position.
using SharpMind.Core.Quantization;

namespace SharpMind.Cuda;

/// <summary>Host-side description of one decoder layer's tensors (GGUF-layout bytes, fp32 vectors).</summary>
public sealed record CudaLayerWeights(byte[] Wq, byte[] Wk, byte[] Wv, byte[] Wo, byte[] WGateUp, byte[] WDown,
    float[] Norm1, float[] Norm2, float[]? QNorm = null, float[]? KNorm = null,
    float[]? Bq = null, float[]? Bk = null, float[]? Bv = null, float[]? Bo = null, float[]? BGateUp = null, float[]? BDown = null);

public sealed record CudaDecoderConfig(int Layers, int Hidden, int Heads, int KvHeads, int HeadDim, int Ffn, int Vocab, int MaxSeq,
    float Eps, float RopeTheta, bool Neox, bool QkNorm, QuantDType Dtype, QuantDType? DownDtype = null,
    QuantDType HeadDtype = QuantDType.Q8_0, int KvKind = CudaKVCache.KindF32);

public sealed unsafe class CudaDecoder : IDisposable
{
    private readonly CudaDecoderConfig _cfg;
    private readonly int _maxBatch;
    private nint _model;
    private readonly List<IDisposable> _owned = [];
    private readonly List<byte[]> _registered = [];
    private readonly DeviceBuffer<int> _tokens, _argmax, _accepted;
    private readonly DeviceBuffer<float> _logits, _uniform, _work;
    private DeviceBuffer<float>? _hidden;
    private readonly nint _lmHead;
    private readonly int _rows;   // rows of logits the buffers hold: max(maxBatch, maxDraft)

    public int Mode { get; set; } = Native.ActQ8;

    public CudaDecoder(CudaDecoderConfig cfg, IReadOnlyList<CudaLayerWeights> layers, byte[] embedding, float[] finalNorm,
                       int maxBatch, int maxDraft = 8)
    {
        if (layers.Count != cfg.Layers) throw new ArgumentException("layer count differs from the configuration");
        (_cfg, _maxBatch) = (cfg, maxBatch);
        int L = cfg.Layers, qDim = cfg.Heads * cfg.HeadDim, kvDim = cfg.KvHeads * cfg.HeadDim;
        var down = cfg.DownDtype ?? cfg.Dtype;

        nint Reg(byte[] raw, QuantDType dt, int n, int k) { _registered.Add(raw); return CudaBackend.Register(raw, dt, n, k); }
        nint Vec(float[]? v)
        {
            if (v is null) return 0;
            var b = new DeviceBuffer<float>(v);
            _owned.Add(b);
            return b.Pointer;
        }

        var wq = new nint[L]; var wk = new nint[L]; var wv = new nint[L]; var wo = new nint[L]; var wgu = new nint[L]; var wd = new nint[L];
        var n1 = new nint[L]; var n2 = new nint[L]; var qn = new nint[L]; var kn = new nint[L];
        var bq = new nint[L]; var bk = new nint[L]; var bv = new nint[L]; var bo = new nint[L]; var bgu = new nint[L]; var bd = new nint[L];
        bool anyBias = false;
        for (int i = 0; i < L; i++)
        {
            var w = layers[i];
            wq[i] = Reg(w.Wq, cfg.Dtype, qDim, cfg.Hidden);
            wk[i] = Reg(w.Wk, cfg.Dtype, kvDim, cfg.Hidden);
            wv[i] = Reg(w.Wv, cfg.Dtype, kvDim, cfg.Hidden);
            wo[i] = Reg(w.Wo, cfg.Dtype, cfg.Hidden, qDim);
            wgu[i] = Reg(w.WGateUp, cfg.Dtype, 2 * cfg.Ffn, cfg.Hidden);
            wd[i] = Reg(w.WDown, down, cfg.Hidden, cfg.Ffn);
            n1[i] = Vec(w.Norm1); n2[i] = Vec(w.Norm2); qn[i] = Vec(w.QNorm); kn[i] = Vec(w.KNorm);
            bq[i] = Vec(w.Bq); bk[i] = Vec(w.Bk); bv[i] = Vec(w.Bv); bo[i] = Vec(w.Bo); bgu[i] = Vec(w.BGateUp); bd[i] = Vec(w.BDown);
            anyBias |= (bq[i] | bk[i] | bv[i] | bo[i] | bgu[i] | bd[i]) != 0;
        }
        _lmHead = Reg(embedding, cfg.HeadDtype, cfg.Vocab, cfg.Hidden);

        fixed (nint* pwq = wq, pwk = wk, pwv = wv, pwo = wo, pwgu = wgu, pwd = wd, pn1 = n1, pn2 = n2, pqn = qn, pkn = kn,
                     pbq = bq, pbk = bk, pbv = bv, pbo = bo, pbgu = bgu, pbd = bd)
        {
            var d = new SmcModelDesc
            {
                NLayers = L, Hidden = cfg.Hidden, NHeads = cfg.Heads, NKvHeads = cfg.KvHeads, HeadDim = cfg.HeadDim, Ffn = cfg.Ffn,
                Vocab = cfg.Vocab, MaxSeq = cfg.MaxSeq, Eps = cfg.Eps, RopeTheta = cfg.RopeTheta,
                Neox = cfg.Neox ? 1 : 0, QkNorm = cfg.QkNorm ? 1 : 0,
                Wq = pwq, Wk = pwk, Wv = pwv, Wo = pwo, Wgu = pwgu, Wdown = pwd,
                Norm1 = pn1, Norm2 = pn2, QNorm = pqn, KNorm = pkn,
                FinalNorm = Vec(finalNorm), LmHead = _lmHead,
                Bq = anyBias ? pbq : null, Bk = anyBias ? pbk : null, Bv = anyBias ? pbv : null,
                Bo = anyBias ? pbo : null, Bgu = anyBias ? pbgu : null, Bdown = anyBias ? pbd : null,
                KvDtype = cfg.KvKind,
            };
            Native.Check(CudaBackend.Ctx, Native.smc_model_create(CudaBackend.Ctx, in d, maxBatch, out _model));   // the arrays are copied
        }
        _rows = Math.Max(maxBatch, maxDraft + 1);
        _tokens = new DeviceBuffer<int>(Math.Max(_rows, 1024));
        _argmax = new DeviceBuffer<int>(_rows);
        _accepted = new DeviceBuffer<int>(1);
        _logits = new DeviceBuffer<float>((long)_rows * cfg.Vocab);
        _uniform = new DeviceBuffer<float>(_rows);
        _work = new DeviceBuffer<float>((long)_rows * (cfg.Vocab + cfg.Hidden));
    }

    /// <summary>ForwardLastLogits over a prompt (one sequence, cache slot <paramref name="seq"/>), fed in chunks;
    /// returns the greedy pick after the last token. Logits of that token stay in <see cref="LogitsPointer"/> row 0.</summary>
    public int Prefill(ReadOnlySpan<int> prompt, int seq = 0, int pos = 0, int chunk = 1024)
    {
        if (prompt.IsEmpty) throw new ArgumentException("empty prompt");
        chunk = (int)Math.Min(chunk, _tokens.Length);
        for (int start = 0; start < prompt.Length; start += chunk)
        {
            var part = prompt.Slice(start, Math.Min(chunk, prompt.Length - start));
            _tokens.Upload(part);
            Native.Check(CudaBackend.Ctx, Native.smc_forward_last_logits(CudaBackend.Ctx, _model, _tokens.Pointer, part.Length, seq,
                                                                        pos + start, Mode, _logits.Pointer, _argmax.Pointer, 0));
        }
        Span<int> pick = stackalloc int[1];
        _argmax.Download(pick);
        return pick[0];
    }

    /// <summary>One new token per sequence at position <paramref name="pos"/>; greedy picks into <paramref name="next"/>.</summary>
    public void Step(ReadOnlySpan<int> tokens, int pos, Span<int> next)
    {
        if (tokens.Length > _maxBatch || next.Length < tokens.Length) throw new ArgumentOutOfRangeException(nameof(tokens));
        _tokens.Upload(tokens);
        Native.Check(CudaBackend.Ctx, Native.smc_decode_step(CudaBackend.Ctx, _model, _tokens.Pointer, tokens.Length, pos, Mode,
                                                            _logits.Pointer, _argmax.Pointer, 0));
        _argmax.Download(next[..tokens.Length]);
    }

    /// <summary>Sampler.Sample on the logits of the last Step / Prefill (rows = sequences). The uniform numbers come from the
    /// caller's Random (one NextSingle() per row), so a seeded run draws the stream it would draw on the CPU.</summary>
    public void Sample(int rows, SmcSampling cfg, ReadOnlySpan<float> uniform, Span<int> tokens,
                       ReadOnlySpan<int> recentIds = default, int window = 0, float repetitionPenalty = 1f)
    {
        if (rows > _rows) throw new ArgumentOutOfRangeException(nameof(rows));
        if (window > 0 && repetitionPenalty != 1f)
        {
            using var ids = new DeviceBuffer<int>(recentIds[..(rows * window)]);
            Native.Check(CudaBackend.Ctx, Native.smc_repetition_penalty_dev(CudaBackend.Ctx, _logits.Pointer, rows, _cfg.Vocab, ids.Pointer,
                                                                           window, repetitionPenalty, 0));
        }
        if (cfg.Temperature > 0f) _uniform.Upload(uniform[..rows]);
        Native.Check(CudaBackend.Ctx, Native.smc_sample_dev(CudaBackend.Ctx, _logits.Pointer, rows, _cfg.Vocab, in cfg, _uniform.Pointer,
                                                           _work.Pointer, _argmax.Pointer, 0));
        _argmax.Download(tokens[..rows]);
    }

    /// <summary>Transformer.Forward(draft): logits and greedy pick for every draft position (MedusaGenerator.cs:259);
    /// returns the accepted count of MedusaGenerator.cs:275-283. Roll-back = the caller's next pos is pos + accepted.</summary>
    public int VerifyDraft(ReadOnlySpan<int> draft, int pos, Span<int> picks, int seq = 0)
    {
        if (draft.Length > _rows) throw new ArgumentOutOfRangeException(nameof(draft));
        _hidden ??= new DeviceBuffer<float>((long)_rows * _cfg.Hidden);
        _tokens.Upload(draft);
        Native.Check(CudaBackend.Ctx, Native.smc_forward_logits(CudaBackend.Ctx, _model, _tokens.Pointer, draft.Length, seq, pos, Mode,
                                                               _logits.Pointer, _argmax.Pointer, _hidden.Pointer, 0));
        Native.Check(CudaBackend.Ctx, Native.smc_verify_greedy_dev(CudaBackend.Ctx, _argmax.Pointer, _tokens.Pointer, draft.Length - 1,
                                                                  _accepted.Pointer, 0));
        _argmax.Download(picks[..draft.Length]);
        Span<int> acc = stackalloc int[1];
        _accepted.Download(acc);
        return acc[0];
    }

    /// <summary>MedusaHeads.Predict from the final-normed hidden row <paramref name="row"/> of the last VerifyDraft.</summary>
    public void MedusaPredict(int row, DeviceBuffer<float> headWeights, DeviceBuffer<float> headBiases, Span<int> outputTokens)
    {
        if (_hidden is null) throw new InvalidOperationException("MedusaPredict needs the hidden rows of a VerifyDraft call");
        int k = outputTokens.Length;
        if (k > _rows) throw new ArgumentOutOfRangeException(nameof(outputTokens));
        Native.Check(CudaBackend.Ctx, Native.smc_medusa_predict_dev(CudaBackend.Ctx, _hidden.Pointer + (nint)((long)row * _cfg.Hidden * sizeof(float)),
                                                                   headWeights.Pointer, headBiases.Pointer, k, _cfg.Hidden, _lmHead,
                                                                   _work.Pointer, _argmax.Pointer, 0));
        _argmax.Download(outputTokens);
    }

    /// <summary>Device pointer of the logits [rows, vocab] of the last call.</summary>
    public nint LogitsPointer => _logits.Pointer;

    public void ReadLogits(int row, Span<float> dst) => _logits.Download(dst[.._cfg.Vocab], (long)row * _cfg.Vocab);

    public void Dispose()
    {
        if (_model != 0) { Native.smc_model_destroy(CudaBackend.Ctx, _model); _model = 0; }
        foreach (var raw in _registered) CudaBackend.Release(raw);
        foreach (var b in _owned) b.Dispose();
        _tokens.Dispose(); _argmax.Dispose(); _accepted.Dispose(); _logits.Dispose(); _uniform.Dispose(); _work.Dispose();
        _hidden?.Dispose();
    }
}
