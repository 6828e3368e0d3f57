"""The benchmark configurations as parity cases against the oracle (seeded N(0,1) inputs of each configuration's
shape; a subset of layers where the CPU oracle would otherwise take minutes)."""
import numpy as np
import pytest

from itak_torch_rebuild_b200 import CudaCompute, KvDtype, PositionCache
from oracle import oracle as orc

from kvparity import assert_attention_close, assert_view_equal, stored

pytestmark = pytest.mark.gpu


def test_config1_tinyllama_prefill_then_decode_f32():
    """22 layers, 32 query / 4 KV heads, head dim 64, f32 cache, batch 1: prefill 512 tokens, then 64 decode steps
    of one token.  Q/K/V ~ N(0,1) from seed 0, RoPE theta 10000 (adjacent pairs, the llama family's pairing,
    crates/arch-llama/src/model.rs:361-391) applied before the append, scale 1/sqrt(64), causal.  Every layer runs
    on the device; layers 0, 9 and 21 are checked row by row against the oracle (tolerance 1e-4 of the norm), and
    their cache contents bit for bit."""
    layers, hq, hkv, d, prefill, steps, theta = 22, 32, 4, 64, 512, 64, 10000.0
    checked = (0, 9, 21)
    gpu = CudaCompute(layers, hq, hkv, d, n_slots=1, max_context=prefill + steps, chunk_cap=prefill,
                      kv_dtype=KvDtype.F32)
    ref = orc.KvCache([orc.GLOBAL] * layers, hkv, d)
    rng = np.random.default_rng(0)
    pos = PositionCache()

    def forward(rows):
        start = pos.position()
        for layer in range(layers):
            q = rng.standard_normal((rows, hq * d)).astype(np.float32)
            k = rng.standard_normal((rows, hkv * d)).astype(np.float32)
            v = rng.standard_normal((rows, hkv * d)).astype(np.float32)
            q = orc.rope_rows(q, hq, d, start, theta).reshape(rows, -1)
            k = orc.rope_rows(k, hkv, d, start, theta).reshape(rows, -1)
            got = gpu.attention(layer, q, k, v, pos)
            assert np.all(np.isfinite(got))
            if layer in checked:
                ref.append_rows(layer, k, v, start)
                want = orc.gqa_attention(q, rows, hq, list(range(start, start + rows)), ref.view(layer))
                assert_attention_close(got, want, hq, d, KvDtype.F32, f"layer {layer} rows {start}..{start + rows}")
        pos.advance(rows)

    forward(prefill)
    for _ in range(steps):
        forward(1)
    assert pos.position() == prefill + steps
    for layer in range(layers):
        assert gpu.next_position(layer) == prefill + steps
    for layer in checked:
        assert_view_equal(gpu, ref, layer, KvDtype.F32)


def test_config2_single_sequence_decode_f16():
    """32 layers, 32 query / 8 KV heads, head dim 128, f16 cache, context 4096 prefilled with seeded N(0,1) K/V,
    then 128 decode steps of append + attention, RoPE theta 500000.  All layers run on the device; layers 0 and
    31 are checked against the oracle at steps 0, 1, 64 and 127 (tolerance 2e-3 of the norm) and their caches bit
    for bit at the end."""
    layers, hq, hkv, d, ctx, steps, theta = 32, 32, 8, 128, 4096, 128, 500000.0
    checked, check_steps = (0, 31), (0, 1, 64, 127)
    dtype = KvDtype.F16
    gpu = CudaCompute(layers, hq, hkv, d, n_slots=1, max_context=ctx + steps, chunk_cap=1, kv_dtype=dtype)
    ref = orc.KvCache([orc.GLOBAL] * layers, hkv, d)
    rng = np.random.default_rng(0)
    for layer in range(layers):
        k = rng.standard_normal((ctx, hkv * d)).astype(np.float32)
        v = rng.standard_normal((ctx, hkv * d)).astype(np.float32)
        if layer in checked:
            k = orc.rope_rows(k, hkv, d, 0, theta).reshape(ctx, -1)
            ref.append_rows(layer, stored(k, dtype), stored(v, dtype), 0)
        gpu.append_rows(layer, k, v, 0)
    pos = PositionCache()
    pos.advance(ctx)
    worst = 0.0
    for step in range(steps):
        p = pos.position()
        for layer in range(layers):
            q = rng.standard_normal(hq * d).astype(np.float32)
            k = rng.standard_normal(hkv * d).astype(np.float32)
            v = rng.standard_normal(hkv * d).astype(np.float32)
            if layer in checked:
                q = orc.rope_rows(q, hq, d, p, theta).reshape(-1)
                k = orc.rope_rows(k, hkv, d, p, theta).reshape(-1)
            got = gpu.attention(layer, q, k, v, pos)
            if layer in checked:
                ref.append(layer, stored(k, dtype), stored(v, dtype), p)
                if step in check_steps:
                    want = orc.gqa_attention(q, 1, hq, [p], ref.view(layer))
                    worst = max(worst, assert_attention_close(got, want, hq, d, dtype, f"step {step} layer {layer}"))
        pos.advance(1)
    assert worst < 1e-4, "the hi/lo tensor-core products should sit far inside the tolerance"
    for layer in checked:
        assert_view_equal(gpu, ref, layer, dtype)


def test_config3_continuous_batching_with_retire_and_refill():
    """16 resident slots with seeded context lengths uniform in [256, 8192], 32 query / 8 KV heads, head dim 128,
    f16 cache: every step appends one token per slot and attends; slot i is retired and refilled with a new seeded
    prompt (reset + bulk append) at steps = 4 i (mod 64).  Two layers on the device; sampled (step, slot) outputs
    and, at the end, sampled slots' caches are checked against per-slot oracle caches."""
    layers, hq, hkv, d, slots_n, steps = 2, 32, 8, 128, 16, 70
    dtype = KvDtype.F16
    rng = np.random.default_rng(0)
    gpu = CudaCompute(layers, hq, hkv, d, n_slots=slots_n, max_context=8192 + steps + 8, chunk_cap=1, kv_dtype=dtype)
    tracked = (0, 5, 11, 15)  # slots mirrored by an oracle cache
    refs = {s: orc.KvCache([orc.GLOBAL] * layers, hkv, d) for s in tracked}
    lens = [0] * slots_n

    def fill(slot):
        n = int(rng.integers(256, 8193))
        for layer in range(layers):
            k = rng.standard_normal((n, hkv * d)).astype(np.float32)
            v = rng.standard_normal((n, hkv * d)).astype(np.float32)
            gpu.append_rows(layer, k, v, 0, slot=slot)
            if slot in refs:
                refs[slot].append_rows(layer, stored(k, dtype), stored(v, dtype), 0)
        lens[slot] = n

    for slot in range(slots_n):
        fill(slot)
    refills = 0
    for step in range(steps):
        for slot in range(slots_n):
            if step > 0 and step % 64 == (4 * slot) % 64:
                gpu.reset(slot=slot)
                if slot in refs:
                    refs[slot] = orc.KvCache([orc.GLOBAL] * layers, hkv, d)
                fill(slot)
                refills += 1
        order = list(range(slots_n))
        for layer in range(layers):
            q = rng.standard_normal((slots_n, hq * d)).astype(np.float32)
            k = rng.standard_normal((slots_n, hkv * d)).astype(np.float32)
            v = rng.standard_normal((slots_n, hkv * d)).astype(np.float32)
            got = gpu.attention_batch(layer, order, lens, 1, q, k, v).reshape(slots_n, -1)
            for slot in tracked:
                refs[slot].append(layer, stored(k[slot], dtype), stored(v[slot], dtype), lens[slot])
                if step % 9 == slot % 9:
                    want = orc.gqa_attention(q[slot], 1, hq, [lens[slot]], refs[slot].view(layer))
                    assert_attention_close(got[slot], want, hq, d, dtype, f"step {step} slot {slot} layer {layer}")
        for slot in range(slots_n):
            lens[slot] += 1
    assert refills >= slots_n
    for slot in tracked:
        for layer in range(layers):
            assert gpu.next_position(layer, slot=slot) == lens[slot]
        assert_view_equal(gpu, refs[slot], 1, dtype, slot=slot)


@pytest.mark.parametrize("hq,hkv", [(64, 8), (8, 1)])
def test_config5_long_context_decode_at_full_context(hq, hkv):
    """The long-context configuration's per-layer shape at its full size - batch 8, context 32768, head dim 128, f16
    cache - with all 8 KV heads (one GPU holding the whole layer: 1 GiB per launch, the equal-run plan) and with one KV
    head (what one of 8 GPUs holds: 128 MiB, the cell-aligned plan with the parts summed in L2), through the
    replayable decode loop the bench uses.  The cache is prefilled on the device with seeded N(0,1) rows; the oracle
    is fed what the device holds (read back through the view) for two of the eight sequences and checked on two
    steps: attention to 2e-3 of the norm, and the rows the steps stored bit for bit."""
    import torch

    from kvparity import as_f32, attention_error

    d, seqs, ctx, steps, layers = 128, 8, 32768, 2, 1
    dtype = KvDtype.F16
    dev = torch.device("cuda", 0)
    gpu = CudaCompute(layers, hq, hkv, d, n_slots=seqs, max_context=ctx + 8, chunk_cap=1, kv_dtype=dtype)
    gen = torch.Generator(device=dev)
    gen.manual_seed(5)
    slots = list(range(seqs))
    kb = torch.empty((seqs, 4096, hkv * d), device=dev)
    vb = torch.empty_like(kb)
    for at in range(0, ctx, 4096):
        kb.normal_(generator=gen)
        vb.normal_(generator=gen)
        gpu.append_rows_device(0, slots, [at] * seqs, 4096, kb.data_ptr(), vb.data_ptr())
    torch.cuda.synchronize()
    sampled = (0, 5)
    refs = {}
    for s in sampled:
        first, k, v = gpu.view(0, slot=s)
        assert first == 0 and k.shape[0] == ctx
        refs[s] = orc.KvCache([orc.GLOBAL], hkv, d)
        refs[s].restore_bulk(0, 0, as_f32(k, dtype), as_f32(v, dtype))
    q = torch.randn((steps, seqs, hq * d), device=dev, generator=gen)
    kn = torch.randn((steps, seqs, hkv * d), device=dev, generator=gen)
    vn = torch.randn((steps, seqs, hkv * d), device=dev, generator=gen)
    out = torch.empty((seqs, hq * d), device=dev)
    gpu.resident_begin(slots, steps)
    worst = 0.0
    for step in range(steps):
        gpu.resident_layer(0, q[step].data_ptr(), kn[step].data_ptr(), vn[step].data_ptr(), out.data_ptr())
        gpu.resident_advance()
        gpu.synchronize()
        got = out.cpu().numpy()
        for s in sampled:
            refs[s].append(0, stored(kn[step, s].cpu().numpy(), dtype), stored(vn[step, s].cpu().numpy(), dtype), ctx + step)
            want = orc.gqa_attention(q[step, s].cpu().numpy(), 1, hq, [ctx + step], refs[s].view(0))
            err = attention_error(got[s], want, hq, d)
            assert err <= 2e-3, f"step {step} sequence {s}: {err:.3e}"
            worst = max(worst, err)
    gpu.resident_end(steps)
    assert worst < 1e-5, "f32-grade products should sit far inside the f16-cache tolerance"
    for s in sampled:
        assert_view_equal(gpu, refs[s], 0, dtype, slot=s)
