"""Test-only stand-ins for streamdiffusionv2_b200.ops that run the oracle on CPU tensors, so that
the host logic (slot mirror, model mirror, streaming scheduler, stage transport) can be checked
without a GPU.  The package itself never imports this."""
import torch

from oracle import causal_attention_oracle as orc


def install(monkeypatch):
    from streamdiffusionv2_b200 import ops

    def rope_table_device(freqs, device):
        return freqs

    def rope_kv_append(q, k, v, k_cache, v_cache, table, grid, start_frames, dst_begin, *, q_out=None,
                       index_tensors=None, index_values=None, norm=None):
        assert norm is None, "the fused norm is a CUDA bf16 path; CPU runs apply the module's own norms"
        rq = orc.rope_apply(q, grid, table, start_frames).type_as(v)
        rk = orc.rope_apply(k, grid, table, start_frames).type_as(v)
        n = q.shape[1]
        for b, d in enumerate(dst_begin):
            if d < 0 or d + n > k_cache.shape[1]:
                raise RuntimeError("slot outside the cache")
            k_cache[b, d:d + n] = rk[b]
            v_cache[b, d:d + n] = v[b]
        if index_tensors is not None:
            g, l = index_tensors
            # raw stores: like the kernel, they do not bump the tensors' version counters
            g.data[:len(index_values[0])] = torch.tensor(index_values[0][:g.numel()], dtype=torch.long)
            l.data[:len(index_values[1])] = torch.tensor(index_values[1][:l.numel()], dtype=torch.long)
        return rq

    def attn(q, k_cache, v_cache, seq_lens, *, out=None, softmax_scale=None):
        return orc.attend_cache(q, k_cache, v_cache, seq_lens)

    def cross(q, k, v, *, out=None, softmax_scale=None):
        return orc.cross_attend(q, k, v)

    monkeypatch.setattr(ops, "rope_table_device", rope_table_device)
    monkeypatch.setattr(ops, "rope_kv_append", rope_kv_append)
    monkeypatch.setattr(ops, "attn_kvcache", attn)
    monkeypatch.setattr(ops, "attn_kvcache_simt", attn)
    monkeypatch.setattr(ops, "cross_attn", cross)
