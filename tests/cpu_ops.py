"""A CPU stand-in for the device ops, built from the oracle's arithmetic.  TEST INFRASTRUCTURE: it
lets the host-side schedule code of the engine (which step follows which, when an all-reduce is
waited for, buffer reuse) run on CPU ranks over gloo.  The product never uses it."""
import torch

from oracle import ladder_oracle as lo


class CpuOps:
    name = "cpu-oracle-stand-in"

    @staticmethod
    def embedding(table, idx, out):
        flat = idx.reshape(-1).long()
        out[: flat.numel()] = table[flat]

    @staticmethod
    def add_rmsnorm(residual, add1, add2, weight, eps, residual_out, normed_out, rows, scale=1.0):
        x = residual[:rows]
        if scale != 1.0:
            x = x * scale
        if add1 is not None:
            x = x + add1[:rows]
        if add2 is not None:
            x = x + add2[:rows]
        x = x.clone()
        if residual_out is not None:
            residual_out[:rows] = x
        if normed_out is not None:
            normed_out[:rows] = lo.rmsnorm(x, weight, eps)

    @staticmethod
    def linear(x, w, out, rows, addend=None, workspace=None):
        y = lo.linear(x[:rows], w)
        if addend is not None:
            y = y + addend[:rows]
        out.view(-1, w.shape[0])[:rows] = y

    @staticmethod
    def linear_workspace_bytes(rows, n):
        return 0

    @staticmethod
    def qkv_workspace_bytes(rows, n_head, n_kv, head_dim):
        return 0

    @staticmethod
    def gateup_workspace_bytes(rows, inter):
        return 0

    @staticmethod
    def attn_decode_scratch_bytes(B, n_head, n_kv, head_dim, num_splits):
        return 0

    @staticmethod
    def qkv_rope_kvcache(x, wqkv, table, table_gathered, input_pos, q_out, k_cache, v_cache, B, S, n_head, n_kv,
                         head_dim, workspace):
        rows = B * S
        qkv = lo.linear(x[:rows], wqkv).view(B, S, -1)
        q, k, v = qkv.split([n_head * head_dim, n_kv * head_dim, n_kv * head_dim], dim=-1)
        trows = table[:S] if table_gathered else table[input_pos.long()]
        q = lo.rope(q.reshape(B, S, n_head, head_dim), trows)
        k = lo.rope(k.reshape(B, S, n_kv, head_dim), trows).transpose(1, 2)
        v = v.reshape(B, S, n_kv, head_dim).transpose(1, 2)
        k_cache[:B, :, input_pos.long()] = k
        v_cache[:B, :, input_pos.long()] = v
        q_out[:rows] = q.reshape(rows, n_head * head_dim)

    @staticmethod
    def gateup_swiglu(x, w1, h, rows, workspace):
        h[:rows] = lo.swiglu(lo.linear(x[:rows], w1))

    @staticmethod
    def attention(q, k_cache, v_cache, input_pos, out, B, S, n_head, n_kv, head_dim, scratch, num_splits):
        rows = B * S
        q4 = q[:rows].view(B, S, n_head, head_dim).transpose(1, 2)
        y = lo.attention_core(q4, k_cache, v_cache, input_pos)
        out[:rows] = y.transpose(1, 2).reshape(rows, n_head * head_dim)
