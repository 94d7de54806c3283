"""A stand-in for capi.Context made of the CPU oracle, for tests that run the decoder DRIVERS
(palm-infra_b200/decoder.py) where there is no GPU: the same Python code path -- buffers,
operator sequence, cache handling, gathers between ranks -- with every operator computed by
the oracle on torch CPU tensors.  Test infrastructure only; it implements just the methods the
drivers call."""
import numpy as np
import torch

import oracle_lib as ol


class _Weight:
    def __init__(self, blocks, n, k):
        self.blocks, self.n, self.k = np.ascontiguousarray(blocks), n, k

    def free(self):
        self.blocks = None


def _np(t):
    return t.detach().contiguous().numpy()


class OracleContext:
    def __init__(self):
        self.launches = 0

    def sync(self):
        pass

    def set_stream(self, _):
        pass

    def close(self):
        pass

    def upload_weight(self, blocks, n, k):
        return _Weight(blocks, n, k)

    def matmul(self, w, x, y, m=None, rule=ol.ACT_G128, **_):
        y.copy_(torch.from_numpy(ol.matmul_w4(w.blocks, w.n, w.k, _np(x), rule=rule)))

    def matmul_argmax(self, w, x, tokens, y=None):
        logits = ol.matmul_w4(w.blocks, w.n, w.k, _np(x))
        for r in range(logits.shape[0]):
            tokens[r] = int(ol.argmax_token(logits[r]))
        if y is not None:
            y.copy_(torch.from_numpy(logits))

    def rms_norm(self, x, weight, eps, out):
        out.copy_(torch.from_numpy(ol.rms_norm(_np(x), _np(weight), eps)))

    def add_rms_norm(self, residual, update, weight, eps, out):
        new, normed = ol.add_rms_norm(_np(residual), _np(update), _np(weight), eps)
        residual.copy_(torch.from_numpy(new))
        out.copy_(torch.from_numpy(normed))

    def swiglu(self, merged, out):
        out.copy_(torch.from_numpy(ol.swiglu(_np(merged))))

    def embed_rows(self, table_fp16_as_int16, ids, out):
        table = _np(table_fp16_as_int16).view(np.float16)
        out.copy_(torch.from_numpy(table[_np(ids).astype(np.int64)].astype(np.float32)))

    def qkv_prepare(self, qkv, tokens, heads, kv_heads, dim, q_weight, k_weight, eps, cos, sin,
                    past, q_out, k_cache, v_cache, capacity, past_dev=None):
        if past_dev is not None:
            past = int(past_dev[0])
        a = _np(qkv)
        q_dim, kv_dim = heads * dim, kv_heads * dim
        c, s = _np(cos)[past:past + tokens], _np(sin)[past:past + tokens]
        q = ol.rms_norm(a[:, :q_dim].reshape(tokens * heads, dim), _np(q_weight), eps)
        k = ol.rms_norm(a[:, q_dim:q_dim + kv_dim].reshape(tokens * kv_heads, dim),
                        _np(k_weight), eps)
        q = ol.rope(q.reshape(tokens, heads, dim), c, s, dim)
        k = ol.rope(k.reshape(tokens, kv_heads, dim), c, s, dim)
        v = a[:, q_dim + kv_dim:].reshape(tokens, kv_heads, dim)
        q_out.copy_(torch.from_numpy(q.reshape(tokens, q_dim)))
        k_cache[:, past:past + tokens] = torch.from_numpy(np.ascontiguousarray(k.transpose(1, 0, 2)))
        v_cache[:, past:past + tokens] = torch.from_numpy(np.ascontiguousarray(v.transpose(1, 0, 2)))

    def attention(self, q, k, v, k_cache, v_cache, out, tokens, heads, kv_heads, dim, past,
                  capacity, scale, past_dev=None):
        assert k is None and v is None, "the drivers append through qkv_prepare"
        if past_dev is not None:
            past = int(past_dev[0])
        k_all = np.ascontiguousarray(_np(k_cache)[:, :past + tokens].transpose(1, 0, 2))
        v_all = np.ascontiguousarray(_np(v_cache)[:, :past + tokens].transpose(1, 0, 2))
        got = ol.causal_attention(_np(q).reshape(tokens, heads, dim), k_all, v_all, heads,
                                  kv_heads, past, scale)
        out.copy_(torch.from_numpy(got.reshape(tokens, heads * dim)))

    def moe_forward(self, hidden, router_fp16_as_int16, top_k, intermediate, gate_up, down, out,
                    **_):
        router = _np(router_fp16_as_int16).view(np.float16)
        got = ol.moe_forward(_np(hidden), router, top_k, intermediate, gate_up.blocks,
                             down.blocks, rule=ol.ACT_G32)[0]  # the reference's per-expert rule
        out.copy_(torch.from_numpy(got))

    def moe_expert_outputs(self, hidden, router_fp16_as_int16, top_k, intermediate,
                           gate_up_local, down_local, expert_begin, expert_count, route_out,
                           indices, weights):
        x = _np(hidden)
        logits = ol.router_logits(x, _np(router_fp16_as_int16).view(np.float16))
        idx, w = ol.select_routes(logits, top_k)
        # the local aggregates are indexed from the first expert this rank holds
        routes = ol.expert_route_outputs(x, idx - expert_begin, intermediate,
                                         gate_up_local.blocks, down_local.blocks, expert_count,
                                         rule=ol.ACT_G32)
        route_out.copy_(torch.from_numpy(routes))
        indices.copy_(torch.from_numpy(idx))
        weights.copy_(torch.from_numpy(w))

    def moe_combine(self, route_out, top_k, indices, weights, out):
        out.copy_(torch.from_numpy(ol.moe_combine(_np(route_out), _np(indices), _np(weights))))

    def advance(self, counter, by=1, token=None, history=None):
        at = int(counter[0])
        if token is not None and history is not None and 0 <= at < history.numel():
            history[at] = token[0]
        counter[0] = at + by
