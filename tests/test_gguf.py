"""GGUF reader / writer and GGML block decoders: PyTorch decoders against a scalar reference written from the block
layouts (CPU), and the CUDA decode / direct-to-NVFP4 kernels against the PyTorch decoders (GPU)."""

import struct

import numpy as np
import pytest
import torch

from triune_b200.runtime.gguf_loader import (BLOCK, GGML_F16, GGML_F32, GGML_Q4_0, GGML_Q4_1, GGML_Q4_K, GGML_Q5_0, GGML_Q5_K, GGML_Q6_K,
                                              GGML_Q8_0, TYPE_NAMES, GGUFFile, dequantize_ggml, dequantize_ggml_tensor, ggml_to_nvfp4,
                                              gguf_to_hf_name, hf_config_from_gguf, is_gguf_file, unpermute_llama_qk, write_gguf)

i8=lambda x: x-256 if x>127 else x
def ref_block(b, t):
    h=lambda o: float(np.frombuffer(bytes(b[o:o+2]),dtype='<f2')[0])
    out=[]
    if t==GGML_Q4_0:
        d=h(0); qs=b[2:]; out=[((qs[i]&0xF)-8)*d for i in range(16)]+[((qs[i]>>4)-8)*d for i in range(16)]
    elif t==GGML_Q4_1:
        d,m=h(0),h(2); qs=b[4:]; out=[(qs[i]&0xF)*d+m for i in range(16)]+[(qs[i]>>4)*d+m for i in range(16)]
    elif t==GGML_Q5_0:
        d=h(0); qh=struct.unpack('<I',bytes(b[2:6]))[0]; qs=b[6:]
        out=[(((qs[i]&0xF)|(((qh>>i)&1)<<4))-16)*d for i in range(16)]+[(((qs[i]>>4)|(((qh>>(i+16))&1)<<4))-16)*d for i in range(16)]
    elif t==GGML_Q8_0:
        d=h(0); out=[i8(x)*d for x in b[2:]]
    elif t in (GGML_Q4_K,GGML_Q5_K):
        d,dmin=h(0),h(2); sc=b[4:16]
        def sm(j):
            if j<4: return sc[j]&63, sc[j+4]&63
            return (sc[j+4]&0xF)|((sc[j-4]>>6)<<4), (sc[j+4]>>4)|((sc[j]>>6)<<4)
        if t==GGML_Q4_K:
            q=b[16:]; y=[]
            for j in range(4):
                s1,m1=sm(2*j); s2,m2=sm(2*j+1)
                y+= [d*s1*(q[32*j+l]&0xF)-dmin*m1 for l in range(32)]+[d*s2*(q[32*j+l]>>4)-dmin*m2 for l in range(32)]
            out=y
        else:
            qh=b[16:48]; ql=b[48:]; y=[]
            for j in range(4):
                s1,m1=sm(2*j); s2,m2=sm(2*j+1); u1,u2=1<<(2*j),2<<(2*j)
                y+= [d*s1*((ql[32*j+l]&0xF)+(16 if qh[l]&u1 else 0))-dmin*m1 for l in range(32)]+[d*s2*((ql[32*j+l]>>4)+(16 if qh[l]&u2 else 0))-dmin*m2 for l in range(32)]
            out=y
    elif t==GGML_Q6_K:
        ql,qh=b[0:128],b[128:192]; sc=[i8(x) for x in b[192:208]]; d=h(208); y=[0.0]*256
        for n in range(2):
            for l in range(32):
                i_s=l//16; Q=ql[64*n:]; H=qh[32*n:]; S=sc[8*n:]
                q1=((Q[l]&0xF)|(((H[l]>>0)&3)<<4))-32; q2=((Q[l+32]&0xF)|(((H[l]>>2)&3)<<4))-32
                q3=((Q[l]>>4)|(((H[l]>>4)&3)<<4))-32; q4=((Q[l+32]>>4)|(((H[l]>>6)&3)<<4))-32
                y[128*n+l]=d*S[i_s]*q1; y[128*n+l+32]=d*S[i_s+2]*q2; y[128*n+l+64]=d*S[i_s+4]*q3; y[128*n+l+96]=d*S[i_s+6]*q4
        out=y
    return out
SCALE_OFFS={GGML_Q4_0:[0],GGML_Q4_1:[0,2],GGML_Q5_0:[0],GGML_Q8_0:[0],GGML_Q4_K:[0,2],GGML_Q5_K:[0,2],GGML_Q6_K:[208]}
def random_blocks(t, nb):
    be,bb=BLOCK[t]
    raw=torch.randint(0,256,(nb,bb),dtype=torch.uint8)
    for off in SCALE_OFFS[t]:
        raw[:,off:off+2]=torch.tensor(np.frombuffer(np.random.uniform(0.01,0.1,nb).astype('<f2').tobytes(),dtype=np.uint8).copy()).view(nb,2)
    return raw


@pytest.mark.parametrize("t", list(SCALE_OFFS))
def test_torch_decoders_match_scalar_reference(t):
    np.random.seed(t)
    torch.manual_seed(t)
    be, bb = BLOCK[t]
    raw = random_blocks(t, 6)
    got = dequantize_ggml(raw.reshape(-1), t, 6 * be)
    want = torch.tensor([v for i in range(6) for v in ref_block(raw[i].tolist(), t)])
    assert torch.allclose(got, want, atol=1e-6, rtol=1e-6), TYPE_NAMES[t]


def test_gguf_file_roundtrip_and_name_map(tmp_path):
    torch.manual_seed(0)
    W = {"token_embd.weight": (torch.randn(64, 32), GGML_F16), "blk.0.attn_q.weight": (torch.randn(32, 32), GGML_Q8_0),
         "blk.0.ffn_up.weight": (torch.randn(64, 32), GGML_Q4_0), "output_norm.weight": (torch.randn(32), GGML_F32)}
    meta = {"general.architecture": "llama", "llama.block_count": 1, "llama.attention.head_count": 2, "llama.embedding_length": 32,
            "llama.rope.freq_base": 10000.0, "tokenizer.ggml.tokens": ["a", "b", "c"], "general.name": "unit"}
    p = write_gguf(tmp_path / "m.gguf", W, meta)
    assert is_gguf_file(p) and not is_gguf_file(__file__)
    with GGUFFile(p) as g:
        assert g.metadata["llama.block_count"] == 1 and g.metadata["tokenizer.ggml.tokens"] == ["a", "b", "c"]
        assert g.tensors["blk.0.ffn_up.weight"]["shape"] == (64, 32)
        tol = {GGML_F16: 2e-3, GGML_Q8_0: 3e-2, GGML_Q4_0: 0.5, GGML_F32: 0.0}
        for k, (w, t) in W.items():
            assert (g.tensor(k, dtype=torch.float32) - w).abs().max() <= tol[t], k
        cfg = hf_config_from_gguf(g.metadata)
    assert cfg["hidden_size"] == 32 and cfg["num_attention_heads"] == 2 and cfg["vocab_size"] == 3
    assert gguf_to_hf_name("blk.3.attn_q.weight") == "model.layers.3.self_attn.q_proj.weight"
    assert gguf_to_hf_name("output.weight") == "lm_head.weight" and gguf_to_hf_name("rope_freqs.weight") is None
    w = torch.arange(16.0).view(8, 2)
    u = unpermute_llama_qk(w, 2)
    assert u[:, 0].tolist() == [0, 4, 2, 6, 8, 12, 10, 14]  # interleaved rotary halves of each head are separated


@pytest.mark.gpu
@pytest.mark.parametrize("t", list(SCALE_OFFS) + [GGML_F16])
def test_cuda_decode_kernel_matches_torch(t):
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    np.random.seed(t)
    be, bb = BLOCK[t]
    nb = 4096 // be * 9
    raw = random_blocks(t, nb) if t in SCALE_OFFS else torch.randn(nb).half().view(torch.uint8).view(nb, 2)
    want = dequantize_ggml(raw.reshape(-1), t, nb * be).bfloat16()
    got = dequantize_ggml_tensor(raw.reshape(-1), t, (nb * be,), device="cuda")
    assert torch.equal(got.cpu(), want)


@pytest.mark.gpu
@pytest.mark.parametrize("hadamard", [False, True])
def test_cuda_ggml_to_nvfp4_matches_two_step_path(hadamard):
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from triune_b200.ops import reference as ref

    np.random.seed(3)
    rows, K = 96, 512
    raw = random_blocks(GGML_Q4_K, rows * K // 256).reshape(-1)
    p, s, ts = ggml_to_nvfp4(raw, GGML_Q4_K, rows, K, "cuda", hadamard)
    w = dequantize_ggml(raw, GGML_Q4_K, rows * K).view(rows, K).cuda()
    wr = ref.fwht16(w) if hadamard else w
    p_ref, s_ref, t_ref = ref.nvfp4_quantize(wr)
    assert torch.allclose(ts, t_ref, rtol=1e-5)
    assert (s.view(torch.uint8) != s_ref.view(torch.uint8)).float().mean() < 0.01 and (p != p_ref).float().mean() < 0.02
    deq = ref.nvfp4_dequantize(p, s, ts, torch.float32)
    assert torch.nn.functional.cosine_similarity(deq.flatten(), wr.flatten(), dim=0) > 0.98
