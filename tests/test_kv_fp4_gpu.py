"""NVFP4 key/value pages on the GPU: the append kernel against the host codec, the attention kernels (tiled prefill through
the widened scratch pool, split-KV decode / verify rows) against the fp32 reference over the very values the pages hold."""
import pytest
import torch

from phaseshift_b200.models.qwen35.config import Qwen35Config, tiny_config
from phaseshift_b200.models.qwen35.weights import build_engine_weights, random_hf_weights
from phaseshift_b200.quant.kv_formats import decode_nvfp4_rows, encode_nvfp4_rows, nvfp4_row_bytes
from phaseshift_b200.runtime.batch import SeqRows, StepBatch
from phaseshift_b200.runtime.state import ModelState, StateConfig

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda:0")


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return float((a - b).norm() / (b.norm() + 1e-12))


@pytest.mark.parametrize("D,hq,hkv", [(256, 12, 2), (128, 8, 4)])
def test_nvfp4_pages_append_prefill_and_decode(D, hq, hkv):
    from phaseshift_b200.ops.cuda_ops import CudaOps
    from phaseshift_b200.ops.ref_ops import RefOps
    cfg = Qwen35Config(vocab_size=1024, hidden_size=512, intermediate_size=512, num_hidden_layers=4,
                       num_attention_heads=hq, num_key_value_heads=hkv, head_dim=D)
    cu, ref = CudaOps(cfg, _dev(), max_seq_len=512), RefOps(cfg, _dev())
    mk = lambda kvd, dt: ModelState(cfg, StateConfig(max_slots=2, max_seq_len=512, page_tokens=16, kv_dtype=kvd,
                                                     kv_capacity_tokens=2048), _dev(), dt)
    st_q, st_b, st_r = mk("nvfp4", torch.bfloat16), mk("bf16", torch.bfloat16), mk("bf16", torch.float32)
    li = cfg.attn_layers[0]
    assert st_q.kv_fmt == 2 and st_q.kv[li].k.shape[-1] == nvfp4_row_bytes(D) and st_q.kv[li].k.dtype == torch.uint8
    nb = st_q.max_blocks
    perm = torch.randperm(st_q.num_pages - 1, generator=torch.Generator().manual_seed(3))[:2 * nb] + 1
    for st in (st_q, st_b, st_r):
        st.block_table[0, :nb] = perm[:nb].int().to(_dev())
        st.block_table[1, :nb] = perm[nb:2 * nb].int().to(_dev())
    hf = random_hf_weights(cfg, seed=3, device="cuda")
    aw = build_engine_weights(cfg, lambda n: hf[n], "bf16", "cuda").layers[li].mixer
    g = torch.Generator(device="cuda").manual_seed(21)
    width = 2 * hq * D + 2 * hkv * D

    def pages_to_reference():
        """The fp32 reference state gets exactly the values the 4-bit pages hold."""
        kq = st_q.kv[li]
        st_r.kv[li].k.copy_(decode_nvfp4_rows(kq.k, kq.k_scale, D))
        st_r.kv[li].v.copy_(decode_nvfp4_rows(kq.v, kq.v_scale, D))

    def run(seqs, qkv, bucket):
        n = qkv.shape[0]
        b = StepBatch(bucket, 2, _dev())
        b.fill(seqs); b.upload()
        q_c = cu.attn_prep(qkv, aw, hq, hkv, b, st_q.kv[li], st_q)
        cu.attn_prep(qkv, aw, hq, hkv, b, st_b.kv[li], st_b)
        q_r = ref.attn_prep(qkv.float(), aw, hq, hkv, b, st_r.kv[li], st_r)
        pages_to_reference()
        o_c = cu.paged_attention(q_c, qkv, hq, hkv, b, st_q.kv[li], st_q, b.max_visible)[:n].clone()
        o_r = ref.paged_attention(q_r, qkv.float(), hq, hkv, b, st_r.kv[li], st_r, b.max_visible)[:n]
        torch.cuda.synchronize()
        assert int(st_q.status[0]) == 0 and int(cu.status[0]) == 0
        return o_c, o_r

    # prefill chunks (the tiled kernels over the widened scratch pool): 203 tokens in slot 0 as 150 + 53, 70 tokens in slot 1
    for slot, p0, n in ((0, 0, 150), (0, 150, 53), (1, 0, 70)):
        x = torch.randn(n, width, device="cuda", generator=g).to(torch.bfloat16)
        o_c, o_r = run([SeqRows(slot, p0, [0] * n, ())], x, 512)
        assert _rel_err(o_c, o_r) < 2e-2, (slot, p0, _rel_err(o_c, o_r))

    # the append kernel against the host codec: the bf16 pool holds the values the 4-bit rows were made from
    for which in ("k", "v"):
        src = getattr(st_b.kv[li], which).float()
        rows_h, ts_h = encode_nvfp4_rows(src)
        host = decode_nvfp4_rows(rows_h, ts_h, D)
        devv = decode_nvfp4_rows(getattr(st_q.kv[li], which), getattr(st_q.kv[li], which + "_scale"), D)
        differ = float((host != devv).float().mean())
        assert differ < 1e-3, (which, differ)
        used = src.abs().amax(dim=-1) > 0
        assert int(used.sum()) == (203 + 70) * hkv
        assert _rel_err(devv[used], src[used]) < 0.12, _rel_err(devv[used], src[used])

    # an 8-row block (speculative verification) and the same rows one per step: the split-KV kernel, bit for bit
    x8 = torch.randn(8, width, device="cuda", generator=g).to(torch.bfloat16)
    o8, r8 = run([SeqRows(0, 203, [0] * 8, ())], x8, 16)
    assert _rel_err(o8, r8) < 2e-2, _rel_err(o8, r8)
    for i in range(8):
        o1, _ = run([SeqRows(0, 203 + i, [0], ())], x8[i:i + 1], 16)
        assert torch.equal(o1[0], o8[i]), i
    # two sequences with a row each in one step
    x2 = torch.randn(2, width, device="cuda", generator=g).to(torch.bfloat16)
    o2, r2 = run([SeqRows(1, 70, [0], ()), SeqRows(0, 211, [0], ())], x2, 16)
    assert _rel_err(o2, r2) < 2e-2, _rel_err(o2, r2)


def test_engine_generates_over_nvfp4_pages():
    """Whole model: prefill and graph-replayed decode over 4-bit pages stay close to the same run over bf16 pages."""
    from phaseshift_b200.runtime.engine import Engine
    cfg = tiny_config()
    hf = random_hf_weights(cfg, seed=0)
    ew = build_engine_weights(cfg, lambda n: hf[n], "bf16", "cuda")
    ids = torch.randint(0, cfg.vocab_size, (40,), generator=torch.Generator().manual_seed(5)).tolist()
    logits, forced = {}, []
    for kvd in ("bf16", "nvfp4"):
        eng = Engine(ew, "cuda", StateConfig(max_slots=1, max_seq_len=128, kv_dtype=kvd))
        s = eng.open_sequence()
        _, out = eng.step([SeqRows(s.slot, 0, ids, (len(ids) - 1,))], [s], want_logits=True)
        rows = [out.logits[0].float().clone()]
        for i in range(4):
            if kvd == "bf16":
                forced.append(int(rows[-1].argmax()))          # the 4-bit run is fed the same tokens
            _, out = eng.step([SeqRows(s.slot, s.position, [forced[i]], (0,))], [s], want_logits=True)
            rows.append(out.logits[0].float().clone())
        logits[kvd] = torch.stack(rows)
        assert eng.status_errors == 0 and bool(torch.isfinite(logits[kvd]).all())
    cos = torch.nn.functional.cosine_similarity(logits["bf16"], logits["nvfp4"], dim=1)
    assert float(cos.min()) > 0.9, cos.tolist()
