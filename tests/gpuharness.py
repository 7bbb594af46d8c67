"""A small rig for GPU parity tests that need full control over arena contents, tables and metadata."""
from __future__ import annotations

import numpy as np

import __graft_entry__ as entry
from oracle import psi_oracle as O

pkg = entry.load_package()


def torch_dtype(dtype):
    import torch
    return {pkg.F32: torch.float32, pkg.BF16: torch.bfloat16, pkg.F16: torch.float16}[dtype]


def to_device(values_f32, dtype, device="cuda:0"):
    """f32 numpy -> device tensor of the storage dtype, rounded by the oracle's RNE conversion (bit-identical input
    for both sides)."""
    import torch
    bits = O.encode(np.ascontiguousarray(values_f32, dtype=np.float32), dtype)
    if dtype == pkg.F32:
        return torch.from_numpy(bits.copy()).to(device)
    return torch.from_numpy(bits.view(np.int16).copy()).to(device).view(torch_dtype(dtype))


def bits_to_device(bits, dtype, device="cuda:0"):
    """Storage bits (oracle encoding) -> device tensor of the storage dtype."""
    import torch
    bits = np.ascontiguousarray(bits)
    if dtype == pkg.F32:
        return torch.from_numpy(bits.view(np.float32).copy()).to(device)
    return torch.from_numpy(bits.view(np.int16).copy()).to(device).view(torch_dtype(dtype))


def bits_of(tensor):
    import torch
    t = tensor.detach().contiguous()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16).cpu().numpy().view(np.uint16)
    return t.cpu().numpy()


class Rig:
    def __init__(self, dtype, num_q_heads, num_kv_heads, head_dim, tokens_per_page, scale, layout, max_tokens,
                 arena_f32=None, num_pages=None, plan_mode=0, kernel_mode=0, max_ctas=0, arena_bits=None):
        import torch
        self.torch = torch
        self.dtype, self.hq, self.hkv, self.d, self.p, self.scale = dtype, num_q_heads, num_kv_heads, head_dim, \
            tokens_per_page, scale
        esz = 4 if dtype == pkg.F32 else 2
        self.page_bytes = 2 * num_kv_heads * tokens_per_page * head_dim * esz
        self.page_elems = self.page_bytes // esz
        if arena_bits is not None:
            bits = np.ascontiguousarray(arena_bits).reshape(-1, self.page_elems)
            if dtype == pkg.F32:
                self.arena = torch.from_numpy(bits.copy()).cuda()
            else:
                self.arena = torch.from_numpy(bits.view(np.int16).copy()).cuda().view(torch_dtype(dtype))
        elif arena_f32 is not None:
            self.arena = to_device(np.asarray(arena_f32, dtype=np.float32).reshape(-1, self.page_elems), dtype)
        else:
            self.arena = torch.zeros((num_pages, self.page_elems), dtype=torch_dtype(dtype), device="cuda:0")
        self.num_pages = self.arena.shape[0]
        self.layout = pkg.GQAPageTableLayout(*layout)
        self.olayout = O.Layout(*layout)
        self.ctx = pkg.Context(0, stream=torch.cuda.current_stream().cuda_stream)
        self.pages = pkg.PageArena(self.ctx, self.num_pages, self.page_bytes, device_ptr=self.arena)
        self.table = pkg.GQARequestPageTable(self.ctx, self.layout)
        self.table_host = np.zeros(layout, dtype=np.uint32)
        cfg = pkg.GQAConfig(num_q_heads, num_kv_heads, head_dim, scale, self.page_bytes, dtype, self.layout, max_tokens,
                            plan_mode, kernel_mode, max_ctas)
        self.gqa = pkg.GQA(self.ctx, cfg)

    def set_pages(self, slot, layer, ids):
        """Logical page list of one (slot, layer) row."""
        ids = np.asarray(ids, dtype=np.uint32)
        self.table.write_row(slot, layer, ids)
        self.table_host[slot, layer].reshape(-1)[: len(ids)] = ids

    def arena_bits(self):
        return bits_of(self.arena).reshape(-1)

    def oracle_attention(self, q_tensor, req_slots, positions, layer=0):
        return O.paged_attention(self.arena_bits(), self.dtype, bits_of(q_tensor), req_slots, positions,
                                 self.table_host.reshape(-1), layer, self.olayout, self.hq, self.hkv, self.d,
                                 self.page_bytes, self.scale)

    def close(self):
        self.ctx.sync()
        self.gqa.close()
        self.table.close()
        self.pages.close()
        self.ctx.close()


def flat_metadata(req_slots, token_indices, cu_tokens):
    slots, positions = [], []
    for r, slot in enumerate(req_slots):
        for i in range(cu_tokens[r + 1] - cu_tokens[r]):
            slots.append(slot)
            positions.append(token_indices[r] + i)
    return slots, positions
