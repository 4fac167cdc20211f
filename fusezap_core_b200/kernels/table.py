"""`CudaOps`: the kernel table of the product, hand-written sm_100a kernels called through their C entry points.

Every method checks devices, dtypes and layouts on the host and passes raw pointers and the current CUDA stream to the
library; nothing here computes. A tensor that is not on a CUDA device, a dtype mix the kernels do not take, or a missing
library raises; there is no CPU or library fallback. Kernels that meet bad data (a token outside the table, a position
without a page) set a bit in a device error word instead of faulting; `check_errors()` reads and clears it.
"""
from __future__ import annotations
import ctypes
from ctypes import c_int, c_void_p, c_float, c_longlong

import torch

from .build import load
from .interface import Ops
from .profile import contexts, ideal_linear_bytes

F32, BF16 = 0, 1
_CODE = {torch.float32: F32, torch.bfloat16: BF16}
_STATUS = {1001: "dtype combination not supported", 1002: "shape not supported", 1003: "misaligned operand",
           1004: "size too large for the kernel", 1005: "driver entry point not found", 1006: "tensor map encode failed"}
_DEVICE_ERRORS = {1: "a token id lies outside the embedding table", 2: "a position has no page in its block table",
                  4: "a position lies outside the position tables", 8: "a bounded wait in a kernel gave up",
                  16: "a selected row lies outside the step"}


_ACTIVATIONS = {"tanh": 0, "sigmoid": 1, "silu": 2, "gelu_tanh": 3, "identity": 4}
RGLRU_COOK_ROWS = 4  # recurrent unit: steps whose longest portion is longer compute the recurrence's coefficients in a launch of their own
SINK_MMA_ROWS = 16  # windowed attention with a sink: steps whose longest portion has this many rows go to the tensor-core kernel
LONG_PORTION = 8    # attention: portions of at least this many tokens go to the tile (prefill) kernels
TILE_ROWS = 128     # token rows per tile of those kernels


class KernelError(RuntimeError):
    pass


KEY_TILE = 128            # keys per key tile of the tile kernels
PIECE_MIN_TILES = 8       # a piece of a query tile cut along the keys covers at least this many key tiles
MAX_PIECES = 48           # pieces in a step at most (each has a float32 scratch slot per head)
MAX_CUT_TILES = 16        # query tiles of a step that can be cut


def attention_tiles(portions, n_rows: int, cut_keys: bool = True, heads: int = 32, items_per_entry: int = 16, sms: int = 148):
    """How the attention kernels split a step. `portions`: (row of the block table, rows, first position) per request
    in the step. Returns (entries, cuts, short rows).

    entries: the TILE_ROWS-row query tiles of the portions with at least LONG_PORTION tokens as (block-table row, first
    row within the portion, range), the ones with the most keys first. range -1: the entry covers all keys its rows see.
    A step with few query tiles and many keys behind them (a small portion of a long prompt) would leave most SMs
    without work: where the tiles times `heads` (a block's work is a tile and a head) are fewer than three quarters of
    the SMs and a tile has 2,048 keys and more behind it, or fewer than twice the SMs with 8,192 keys and more, tiles are
    cut along the keys into pieces of equal length, at least PIECE_MIN_TILES key tiles each, range =
    first key tile | key tiles << 16, whose partial results a merge kernel adds up. As many pieces are made as give two
    rounds of items for the SMs (`items_per_entry`: heads, or pairs of heads for the kernel that takes two per block).
    The pieces stand first in the list (their index is their scratch slot) and the pieces of one tile stand together.
    cuts: (first entry, entries) per tile that was cut. short rows: the step's other rows (short portions, single tokens
    and padding), which go to the split-key kernel."""
    tiles, long_rows = [], 0
    for seq_row, n, pos0 in portions:
        if n >= LONG_PORTION:
            long_rows += n
            tiles += [(pos0 + min(r + TILE_ROWS, n), seq_row, r) for r in range(0, n, TILE_ROWS)]
    tiles.sort(key=lambda t: -t[0])
    short = n_rows - long_rows
    key_tiles = [(last - 1) // KEY_TILE + 1 for last, _, _ in tiles]
    total = sum(key_tiles)
    # (measured through the engine at 32 heads and 8 layers: with at least 0.75 items per SM the cuts pay from about
    # 8,192 keys on: a 32,000-token prompt in portions of 768 took 226 ms without them and 198 ms with them, in portions
    # of 1,024 198 and 189 ms; a 7,680-token prompt in portions of 512 38.0 ms without and 38.8 ms with)
    items = len(tiles) * heads
    enough = 2 * PIECE_MIN_TILES if 4 * items < 3 * sms else 8 * PIECE_MIN_TILES
    if not cut_keys or not tiles or items >= 2 * sms or key_tiles[0] < enough or key_tiles[0] >= 1 << 15:
        return [(s, r, -1) for _, s, r in tiles], [], short
    target = min(MAX_PIECES, max(2, (2 * sms) // max(1, items_per_entry)))
    pieces, cuts, whole = [], [], []
    for (_, s, r), kt in zip(tiles, key_tiles):
        n = min(kt // PIECE_MIN_TILES, max(1, round(target * kt / total)))
        if n < 2 or len(pieces) + n > MAX_PIECES or len(cuts) >= MAX_CUT_TILES:
            whole.append((s, r, -1))
            continue
        each = -(-kt // n)
        cuts.append((len(pieces), -(-kt // each)))
        pieces += [(s, r, lo | (min(each, kt - lo) << 16)) for lo in range(0, kt, each)]
    return pieces + whole, cuts, short


class AttentionPlan:
    """What `plan_step` keeps about a step for the attention kernels: the device views of the entry list and of the list
    of tiles cut along the keys, and the counts that size the launches."""
    __slots__ = ("tiles", "n_tiles", "n_short_rows", "cuts", "n_cuts", "n_pieces", "single_tokens")

    def __init__(self, tiles: torch.Tensor | None, n_tiles: int, n_short_rows: int, cuts: torch.Tensor | None = None,
                 n_cuts: int = 0, n_pieces: int = 0, single_tokens: bool = False):
        self.tiles, self.n_tiles, self.n_short_rows = tiles, n_tiles, n_short_rows
        self.cuts, self.n_cuts, self.n_pieces = cuts, n_cuts, n_pieces
        # every portion of the step is one token (a decode step): the kernel for short rows then asks for no portion records
        self.single_tokens = single_tokens


def _p(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


class CudaOps(Ops):
    def __init__(self, dtype: str | torch.dtype, device: str | torch.device = "cuda:0"):
        self.dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}.get(dtype, dtype)
        if self.dtype not in _CODE:
            raise ValueError(f"dtype {dtype!r} is not float32 or bfloat16")
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise KernelError(f"the kernels run on a CUDA device only, not on {self.device}")
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device is available; this engine has no CPU path")
        self.core = load("fzb200_core")
        self.err = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._err_host = torch.zeros(1, dtype=torch.int32, pin_memory=True)
        self.launches = 0
        self._stream_handle = None
        self._scratch_bufs: dict[str, torch.Tensor] = {}
        self._retired: list[torch.Tensor] = []      # outgrown scratch: a captured step may still point at it
        self.tc = None
        if self.dtype == torch.bfloat16:
            self.tc = load("fzb200_tc")      # tcgen05 / TMA kernels
        self.use_tensor_cores = self.tc is not None
        self._attn_tc = self._mix = self._mix_tc = self._latent = self._latent_tc = self._seq = self._seq_tc = self._rows = None   # libraries loaded (and built) when a part first asks for their kernels
        self.prefill_tcgen05 = True        # False: long portions on the mma.sync flash-attention kernel
        self.fuse_swiglu = True            # gate/up product and SwiGLU in one kernel where the sizes allow it
        self.fuse_argmax = True            # lm_head product and argmax in one pass where no logits are asked for
        self.sink_max_runs = 64            # single-token steps over all earlier keys: a row's keys are cut into at most this many runs
        self.fuse_depth_norm = True        # the depth average of a layer's result and the norm that follows in one kernel
        self.fuse_rope = True              # q/k/v product, rotation and cache write in one kernel (few-token steps)
        # 128-row tiles for experts with hundreds of rows: measured slower for the gated product (347 against 319 us at
        # 8,192 pairs x 2,048 x 1,024) and the same for the scatter product (199 against 205 us), so off
        self.grouped_tiles_128 = False
        self.grouped_tensor_cores = True   # products per head and per expert on tensor cores where the sizes allow it
        self.latent_key_cuts = True        # latent attention: few tiles with many keys are cut along the keys
        self.latent_tensor_cores = True    # latent attention on tensor cores where the sizes allow it (bfloat16)
        self.cut_prefill_keys = True       # few query tiles with many keys behind them are cut along the keys
        self._profile = None               # a StepProfile while the engine profiles its steps
        self._meta_rows = None             # meta.seq_row of the step being run, for ops that take no `meta`
        self.split_decode_keys = True      # windowed attention with a sink: steps of single tokens cut a row's keys into runs
        self.sink_tensor_cores = True      # that attention on tensor cores for portions of SINK_MMA_ROWS rows and more (bfloat16)
        # the fewest query heads, and the fewest items of a query tile on the prompt kernel, among the attention layers
        # that `check_attention` has seen (the plan of a step is shared by its layers)
        self._attn_heads = self._attn_items = 0
        self._sms = torch.cuda.get_device_properties(self.device).multi_processor_count

    # ---- plumbing
    @property
    def mix_tc(self):
        """The products per head and per expert on tensor cores (bfloat16)."""
        if self._mix_tc is None:
            self._mix_tc = load("fzb200_mix_tc")
        return self._mix_tc

    @property
    def attn_tc(self):
        """The tensor-core attention kernels over separate keys and values (bfloat16)."""
        if self._attn_tc is None:
            self._attn_tc = load("fzb200_attn_tc")
        return self._attn_tc

    @property
    def latent(self):
        """The general attention over a shared latent cache."""
        if self._latent is None:
            self._latent = load("fzb200_latent")
        return self._latent

    @property
    def latent_tc(self):
        """The tensor-core attention over a shared latent cache (bfloat16)."""
        if self._latent_tc is None:
            self._latent_tc = load("fzb200_latent_tc")
        return self._latent_tc

    @property
    def seq_tc(self):
        """The attention with a window, kept first tokens and a sink on tensor cores (bfloat16, prompt portions)."""
        if self._seq_tc is None:
            self._seq_tc = load("fzb200_seq_tc")
        return self._seq_tc

    @property
    def seq(self):
        """The recurrent scans, the attention with a window, kept first tokens and a sink, the experts' router."""
        if self._seq is None:
            self._seq = load("fzb200_seq")
        return self._seq

    @property
    def rows(self):
        """Depth-averaged layers, the hashed pair embedding, a columnwise activation."""
        if self._rows is None:
            self._rows = load("fzb200_rows")
        return self._rows

    @property
    def mix(self):
        """The kernels of the gated parallel block, the latent attention and the products per head and per expert."""
        if self._mix is None:
            self._mix = load("fzb200_mix")
        return self._mix

    def begin_step(self) -> None:
        """Called by the step function before it launches anything: the kernels of the step all go to the stream that
        is current now (asked for once; it changes when a graph is captured or a caller switches streams)."""
        self._stream_handle = c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        if self._profile is not None:
            self._profile.begin_step()

    def start_profile(self) -> None:
        """From now on a CUDA event is recorded after every launch (see kernels/profile.py)."""
        from .profile import StepProfile
        self._profile = StepProfile(lambda: torch.cuda.Event(enable_timing=True))

    def profile_report(self) -> dict:
        if self._profile is None:
            raise KernelError("start_profile() was not called")
        self._profile.collect(lambda: torch.cuda.synchronize(self.device))
        return self._profile.report()

    def end_step(self) -> None:
        self._stream_handle = None

    def _stream(self) -> c_void_p:
        if self._stream_handle is not None:
            return self._stream_handle
        return c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def _scratch(self, name: str, numel: int, dtype: torch.dtype, zero: bool = False) -> torch.Tensor:
        """A scratch buffer of at least `numel` elements. It only ever grows, and a buffer that was outgrown is kept
        alive, since a captured step that was recorded with it still writes there."""
        buf = self._scratch_bufs.get(name)
        if buf is None or buf.numel() < numel:
            if buf is not None:
                self._retired.append(buf)
            buf = (torch.zeros if zero else torch.empty)(numel, dtype=dtype, device=self.device)
            self._scratch_bufs[name] = buf
        return buf

    def _check(self, status: int, what: str, ideal_bytes: int = 0) -> None:
        self.launches += 1
        if status != 0:
            why = _STATUS.get(status, f"CUDA error {status}")
            raise KernelError(f"{what}: {why}")
        if self._profile is not None:
            self._profile.note(what, ideal_bytes)

    def _want(self, t: torch.Tensor, name: str, dtypes: tuple, dims: int | None = None) -> None:
        if not t.is_cuda:
            raise KernelError(f"{name} is on {t.device}; the kernels take CUDA tensors only")
        if t.dtype not in dtypes:
            raise KernelError(f"{name} has dtype {t.dtype}, expected one of {dtypes}")
        if not t.is_contiguous():
            raise KernelError(f"{name} is not contiguous")
        if dims is not None and t.dim() != dims:
            raise KernelError(f"{name} has {t.dim()} dimensions, expected {dims}")

    def errors_to_host(self) -> None:
        """Enqueues the copy of the error word to pinned memory on the current stream; after the caller's own
        synchronisation `check_errors(copied=True)` reads it without another round trip."""
        self._err_host.copy_(self.err, non_blocking=True)

    def check_errors(self, copied: bool = False) -> None:
        """Raises if any kernel since the last check flagged bad data. copied=False waits for the device first."""
        word = int(self._err_host[0]) if copied else int(self.err.item())
        if word:
            self.err.zero_()
            raise KernelError("a kernel reported: " + "; ".join(m for b, m in _DEVICE_ERRORS.items() if word & b))

    # ---- per-step planning (the step function calls these; it knows nothing of the kernels' tiling)
    def step_extra_ints(self, needs: tuple, max_rows: int, max_segments: int) -> int:
        """int32 this table wants in the step's metadata block for a model whose mixers need `needs`: three per entry of
        the attention tile list (a query tile per TILE_ROWS rows and one more per portion, plus the pieces of tiles cut
        along the keys), two per tile that is cut."""
        if "attention" not in needs:
            return 0
        return 3 * (max_rows // TILE_ROWS + max_segments + MAX_PIECES) + 2 * MAX_CUT_TILES

    def plan_step(self, meta, needs: tuple) -> None:
        """Called when a step has been packed on the host, before its one copy to the device: writes the attention
        kernels' tile list into the block's extra part and keeps the launch sizes in `meta.plan`."""
        # kernels that tile the rows of portions size their grid by the longest portion
        meta.portion_tiles = int(meta.max_portion) if "portions" in needs else 0
        if "latent_attention" in needs:
            # The latent attention takes 64 (row, head) pairs of one portion per block: rows x heads / 64 blocks and at
            # most one more per portion. A step of single tokens may be replayed as a captured graph with other
            # requests in its rows, so it allows one per row.
            single = all(sg.n == 1 for sg in meta.segments)
            meta.latent_extra = meta.n_rows if single else meta.n_segments
        if "attention" not in needs:
            meta.plan = None
            return
        # tiles are cut along the keys only for the kernel that can leave partial results (tcgen05, pages TMA can box)
        page = getattr(meta, "page_size", 0)
        can_cut = self.cut_prefill_keys and self.use_tensor_cores and self.prefill_tcgen05 and \
            (page == 8 or (page > 0 and page % 16 == 0))
        entries, cuts, short = attention_tiles(((sg.seq_row, sg.n, sg.pos0) for sg in meta.segments), meta.n_rows, can_cut,
                                               self._attn_heads or 32, self._attn_items or 16, self._sms)
        n_list = (meta.extra_host.size - 2 * MAX_CUT_TILES) // 3
        host = meta.extra_host[:3 * n_list].reshape(-1, 3)
        host[len(entries):] = -1
        if entries:
            host[:len(entries)] = entries
        host_cuts = meta.extra_host[3 * n_list:].reshape(-1, 2)
        host_cuts[len(cuts):] = 0
        if cuts:
            host_cuts[:len(cuts)] = cuts
        meta.plan = AttentionPlan(meta.extra[:3 * n_list].view(-1, 3), len(entries), short, meta.extra[3 * n_list:].view(-1, 2),
                                  len(cuts), sum(c for _, c in cuts), single_tokens=all(sg.n == 1 for sg in meta.segments))

    def step_signature(self, meta) -> tuple:
        """What, beside the row counts, fixes the kernel launches of a step (two steps that agree in it launch alike)."""
        plan = meta.plan
        latent = (getattr(meta, "latent_extra", 0), getattr(meta, "portion_tiles", 0))
        return (plan.n_tiles, plan.n_short_rows > 0, plan.n_cuts, plan.single_tokens, *latent) if plan is not None else latent

    def check_attention(self, num_heads: int, num_kv_heads: int, head_dim: int) -> None:
        if head_dim % 16:
            raise ValueError(f"head_dim {head_dim} is not a multiple of 16; the attention kernels refuse it")
        if self.core.fz_attn_simt_check(c_int(num_heads), c_int(num_kv_heads), c_int(head_dim)) != 0:
            raise ValueError(f"attention sizes not supported: {num_heads} heads, {num_kv_heads} kv heads, head_dim "
                             f"{head_dim} (need heads % kv_heads == 0 and head_dim <= 512)")
        # (the prompt kernel takes two heads of a kv head per block at head size 128, else one)
        if self.use_tensor_cores:
            self.attn_tc      # built and loaded with the model, not at its first step
        items = num_kv_heads * ((num_heads // num_kv_heads + 1) // 2) if head_dim == 128 else num_heads
        self._attn_heads = min(self._attn_heads or num_heads, num_heads)
        self._attn_items = min(self._attn_items or items, items)

    # ---- kernels
    def embed(self, table, tokens, x, src=None, prev_ids=None, scale: float = 1.0) -> None:
        self._want(table, "embedding table", (torch.float32, torch.bfloat16), 2)
        self._want(tokens, "tokens", (torch.int32,), 1)
        self._want(x, "x", (torch.float32,), 2)
        n, d = x.shape
        if tokens.shape[0] != n or table.shape[1] != d:
            raise KernelError(f"embed: tokens {tuple(tokens.shape)}, table {tuple(table.shape)}, x {tuple(x.shape)}")
        if src is not None:
            self._want(src, "src", (torch.int32,), 1)
            self._want(prev_ids, "prev_ids", (torch.int32,), 1)
        self._check(self.core.fz_embed(_p(table), c_int(_CODE[table.dtype]), _p(tokens), _p(src),
                                       _p(prev_ids if src is not None else None), _p(x), c_int(n), c_int(d),
                                       c_int(table.shape[0]), c_float(scale), _p(self.err), self._stream()), "embed",
                    n * d * (table.element_size() + 4))

    def add_rmsnorm(self, x, delta, weight, eps, h, rows=None, groups: int = 1) -> None:
        self._want(x, "x", (torch.float32,), 2)
        self._want(weight, "norm weight", (torch.float32, torch.bfloat16), 1)
        self._want(h, "h", (torch.float32, torch.bfloat16), 2)
        if delta is not None:
            self._want(delta, "delta", (torch.float32,), 2)
            if delta.shape != x.shape:
                raise KernelError(f"add_rmsnorm: delta {tuple(delta.shape)} vs x {tuple(x.shape)}")
        n_src, d = x.shape
        n_out = n_src
        if rows is not None:
            self._want(rows, "rows", (torch.int32,), 1)
            n_out = rows.shape[0]
        if h.shape != (n_out, d) or weight.shape[0] != d:
            raise KernelError(f"add_rmsnorm: h {tuple(h.shape)}, expected {(n_out, d)}; weight {tuple(weight.shape)}")
        nbytes = n_out * d * (4 + (8 if delta is not None and rows is None else 4 if delta is not None else 0) + h.element_size())
        if groups != 1:
            if groups <= 0 or d % groups:
                raise KernelError(f"add_rmsnorm: a row of {d} values does not split into {groups} equal groups")
            self._check(self.mix.fz_add_rmsnorm_groups(_p(x), _p(delta), _p(weight), c_int(_CODE[weight.dtype]), _p(h),
                                                       c_int(_CODE[h.dtype]), _p(rows), c_int(n_out), c_int(n_src), c_int(d),
                                                       c_int(groups), c_float(eps), _p(self.err), self._stream()),
                        "add_rmsnorm (groups)", nbytes)
            return
        self._check(self.core.fz_add_rmsnorm(_p(x), _p(delta), _p(weight), c_int(_CODE[weight.dtype]), _p(h),
                                             c_int(_CODE[h.dtype]), _p(rows), c_int(n_out), c_int(n_src), c_int(d),
                                             c_float(eps), _p(self.err), self._stream()), "add_rmsnorm",
                    n_out * d * (4 + (8 if delta is not None and rows is None else 4 if delta is not None else 0) + h.element_size()))

    def linear(self, a, w, bias, out) -> None:
        self._want(a, "linear input", (self.dtype,), 2)
        self._want(w, "linear weight", (self.dtype,), 2)
        self._want(out, "linear output", (torch.float32, self.dtype), 2)
        if bias is not None:
            self._want(bias, "linear bias", (torch.float32,), 1)
        m, k = a.shape
        n = w.shape[0]
        if w.shape[1] != k or out.shape != (m, n) or (bias is not None and bias.shape[0] != n):
            raise KernelError(f"linear: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
        self._gemm(a, w, bias, out, m, n, k)

    def _gemm(self, a, w, bias, out, m, n, k) -> None:
        if self.use_tensor_cores and self.tc.fz_gemm_tc_check(_p(a), _p(w), c_int(m), c_int(n), c_int(k)) == 0:
            self._check(self.tc.fz_gemm_tc(
                _p(a), _p(w), _p(bias), _p(out), c_int(_CODE[out.dtype]), c_int(m), c_int(n), c_int(k),
                _p(self.err), self._stream()), "linear (tensor cores)",
                ideal_linear_bytes(m, n, k, 2, 2, out.element_size()))
            return
        self._check(self.core.fz_gemm_simt(_p(a), _p(w), _p(bias), _p(out), c_int(_CODE[a.dtype]),
                                           c_int(_CODE[out.dtype]), c_int(m), c_int(n), c_int(k), self._stream()),
                    "linear", ideal_linear_bytes(m, n, k, a.element_size(), w.element_size(), out.element_size()))

    def pack_gate_up(self, gate, up, gate_bias=None, up_bias=None):
        """Rows in blocks of 128 = [64 gate rows | 64 up rows] of the same 64 features, so that one 128-row tile of the
        tensor-core product holds both halves of its outputs. None when the fused kernel does not apply."""
        i, k = gate.shape
        if not self.use_tensor_cores or not self.fuse_swiglu or gate.dtype != torch.bfloat16 or i % 64 or k % 8:
            return None
        w = torch.stack([gate.view(i // 64, 64, k), up.view(i // 64, 64, k)], 1).reshape(2 * i, k).contiguous()
        b = None
        if gate_bias is not None:
            b = torch.stack([gate_bias.float().view(i // 64, 64), up_bias.float().view(i // 64, 64)], 1).reshape(2 * i).contiguous()
        return (w, b, i)

    def linear_swiglu(self, a, packed, out, activation: str = "silu") -> None:
        w, b, i = packed
        self._want(a, "linear input", (torch.bfloat16,), 2)
        self._want(out, "swiglu output", (torch.bfloat16,), 2)
        m, k = a.shape
        if w.shape != (2 * i, k) or out.shape != (m, i):
            raise KernelError(f"linear_swiglu: a {tuple(a.shape)}, packed {tuple(w.shape)}, out {tuple(out.shape)}")
        self._check(self.tc.fz_gemm_tc_swiglu(_p(a), _p(w), _p(b), _p(out), c_int(m), c_int(i), c_int(k),
                                              c_int(self._gate_kind(activation)), _p(self.err),
                                              self._stream()), "linear_swiglu (tensor cores)",
                    ideal_linear_bytes(m, 2 * i, k, 2, 2, 1))

    def _pool(self, cache, hkv: int, hd: int):
        k, v = cache.keys, cache.values
        for t, name in ((k, "key pool"), (v, "value pool")):
            if not t.is_cuda or t.dtype != self.dtype:
                raise KernelError(f"{name}: device {t.device}, dtype {t.dtype}; expected CUDA {self.dtype}")
            if t.dim() != 4 or t.shape[1] != hkv or t.shape[3] != hd or t.shape[2] != cache.page_size:
                raise KernelError(f"{name} has shape {tuple(t.shape)}, expected (pages, {hkv}, {cache.page_size}, {hd})")
            if t.stride(3) != 1 or t.stride(2) != hd or t.stride(1) != cache.page_size * hd:
                raise KernelError(f"{name} has strides {t.stride()}: a page's heads must be contiguous")
        if k.stride(0) != v.stride(0):
            raise KernelError("key and value pools have different page strides")
        return k, v, k.stride(0)

    def rope_kv_write(self, qkv, cos, sin, meta, cache, q_out, num_heads, num_kv_heads, head_dim) -> None:
        self._want(qkv, "qkv", (torch.float32,), 2)
        self._want(cos, "cos table", (torch.float32,), 2)
        self._want(sin, "sin table", (torch.float32,), 2)
        self._want(q_out, "q", (self.dtype,), 2)
        n = qkv.shape[0]
        if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim or q_out.shape != (n, num_heads * head_dim) \
                or cos.shape[1] != head_dim // 2 or sin.shape != cos.shape:
            raise KernelError(f"rope_kv_write: qkv {tuple(qkv.shape)}, q {tuple(q_out.shape)}, cos {tuple(cos.shape)}")
        k, v, page_stride = self._pool(cache, num_kv_heads, head_dim)
        table = meta.table(cache.group)
        self._check(self.core.fz_rope_kv_write(
            _p(qkv), _p(cos), _p(sin), _p(meta.pos), _p(meta.seq_row), _p(table), c_int(table.shape[1]), _p(k), _p(v),
            c_longlong(page_stride), c_int(cache.page_size), c_int(1 if cache.write else 0), _p(q_out),
            c_int(_CODE[self.dtype]), c_int(n), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim),
            c_int(cos.shape[0]), _p(self.err), self._stream()), "rope_kv_write")

    def linear_rope_kv_write(self, a, w, bias, cos, sin, meta, cache, q_out, num_heads, num_kv_heads, head_dim) -> bool:
        m, k = a.shape
        if not (self.use_tensor_cores and self.fuse_rope and self.dtype == torch.bfloat16) or \
                self.tc.fz_gemm_tc_qkv_rope_check(c_int(m), c_int(head_dim)) != 0 or \
                self.tc.fz_gemm_tc_check(_p(a), _p(w), c_int(m), c_int(w.shape[0]), c_int(k)) != 0:
            return False
        self._want(a, "linear input", (torch.bfloat16,), 2)
        self._want(w, "linear weight", (torch.bfloat16,), 2)
        self._want(cos, "cos table", (torch.float32,), 2)
        self._want(sin, "sin table", (torch.float32,), 2)
        self._want(q_out, "q", (torch.bfloat16,), 2)
        if bias is not None:
            self._want(bias, "linear bias", (torch.float32,), 1)
        n = (num_heads + 2 * num_kv_heads) * head_dim
        if w.shape != (n, k) or q_out.shape != (m, num_heads * head_dim) or cos.shape[1] != head_dim // 2 \
                or sin.shape != cos.shape or (bias is not None and bias.shape[0] != n):
            raise KernelError(f"linear_rope_kv_write: a {tuple(a.shape)}, w {tuple(w.shape)}, q {tuple(q_out.shape)}, "
                              f"cos {tuple(cos.shape)}")
        kp, vp, page_stride = self._pool(cache, num_kv_heads, head_dim)
        table = meta.table(cache.group)
        self._check(self.tc.fz_gemm_tc_qkv_rope(
            _p(a), _p(w), _p(bias), c_int(m), c_int(k), _p(cos), _p(sin), _p(meta.pos), _p(meta.seq_row), _p(table),
            c_int(table.shape[1]), _p(kp), _p(vp), c_longlong(page_stride), c_int(cache.page_size),
            c_int(1 if cache.write else 0), _p(q_out), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim),
            c_int(cos.shape[0]), _p(self.err), self._stream()), "linear_rope_kv_write (tensor cores)",
            ideal_linear_bytes(m, n, k, 2, 2, 2))
        return True

    def linear_argmax(self, a, w, bias, out) -> bool:
        m, k = a.shape
        n = w.shape[0]
        if not (self.use_tensor_cores and self.fuse_argmax and self.dtype == torch.bfloat16) or \
                self.tc.fz_gemm_tc_argmax_check(c_int(m), c_int(n), c_int(k)) != 0 or \
                self.tc.fz_gemm_tc_check(_p(a), _p(w), c_int(m), c_int(n), c_int(k)) != 0:
            return False
        self._want(a, "linear input", (torch.bfloat16,), 2)
        self._want(w, "linear weight", (torch.bfloat16,), 2)
        self._want(out, "argmax output", (torch.int32,), 1)
        if bias is not None:
            self._want(bias, "linear bias", (torch.float32,), 1)
        if w.shape[1] != k or out.shape[0] != m or (bias is not None and bias.shape[0] != n):
            raise KernelError(f"linear_argmax: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
        need = m * ((n + 127) // 128)
        tile_val = self._scratch("lm_head tile maxima", need, torch.float32)
        tile_idx = self._scratch("lm_head tile indices", need, torch.int32)
        self._check(self.tc.fz_gemm_tc_argmax(_p(a), _p(w), _p(bias), c_int(m), c_int(n), c_int(k), _p(tile_val),
                                              _p(tile_idx), _p(out), _p(self.err), self._stream()),
                    "linear_argmax (tensor cores)", ideal_linear_bytes(m, n, k, 2, 2, 0))
        self.launches += 1     # the reduction over the tiles
        return True

    def paged_attention(self, q, cache, meta, out, num_heads, num_kv_heads, head_dim, scale, window) -> None:
        self._want(q, "q", (self.dtype,), 2)
        self._want(out, "attention output", (self.dtype,), 2)
        n = q.shape[0]
        if q.shape[1] != num_heads * head_dim or out.shape != q.shape:
            raise KernelError(f"paged_attention: q {tuple(q.shape)}, out {tuple(out.shape)}")
        k, v, page_stride = self._pool(cache, num_kv_heads, head_dim)
        table = meta.table(cache.group)
        self._attention(q, k, v, page_stride, cache, meta, table, out, n, num_heads, num_kv_heads, head_dim, scale, window)

    def _attention(self, q, k, v, page_stride, cache, meta, table, out, n, hq, hkv, hd, scale, window) -> None:
        # least bytes: keys and values (a short row reads every key it sees; the rows of a long portion share them, so its
        # keys count once), the queries and the output
        kv = kv_tiles = 0
        if self._profile is not None:
            segs = list(getattr(meta, "segments", ()))
            key_bytes = hkv * hd * 2 * k.element_size()
            kv = contexts([sg for sg in segs if sg.n < LONG_PORTION]) * key_bytes + 2 * n * hq * hd * q.element_size()
            kv_tiles = sum(sg.pos0 + sg.n for sg in segs if sg.n >= LONG_PORTION) * key_bytes
        if self.use_tensor_cores and self.attn_tc.fz_attn_decode_check(c_int(hq), c_int(hkv), c_int(hd)) == 0:
            plan = meta.plan
            if plan is None:
                raise KernelError("paged_attention: the step was not planned (plan_step with the need 'attention')")
            if plan.n_short_rows > 0:
                # rows of short portions and decoded tokens: split over key partitions, partials in float32 scratch
                parts = self.attn_tc.fz_attn_partitions(c_int(meta.max_context))
                need = n * hq * parts * (hd + 2)
                part_o = self._scratch("attention partials", need, torch.float32)
                part_ml = part_o[n * hq * parts * hd:]
                self._check(self.attn_tc.fz_attn_decode(
                    _p(q), _p(k), _p(v), _p(meta.pos), _p(meta.seq_row), _p(meta.seg), _p(table), c_int(table.shape[1]),
                    c_longlong(page_stride), c_int(cache.page_size), _p(out), _p(part_o), _p(part_ml), c_int(n),
                    c_int(hq), c_int(hkv), c_int(hd), c_float(scale), c_int(window), c_int(meta.max_context),
                    c_int(LONG_PORTION), c_int(1 if plan.single_tokens else 0), c_int(k.shape[0]), _p(self.err), self._stream()),
                    "paged_attention (decode)", kv)
                self.launches += 1    # the combine kernel
            if plan.n_tiles > 0 and self.prefill_tcgen05 and \
                    self.attn_tc.fz_attn_prefill_tc_check(c_int(hq), c_int(hkv), c_int(hd), c_int(cache.page_size)) == 0:
                # rows of long portions on the tcgen05 flash-attention kernel; the pieces of tiles that the plan cut along
                # the keys leave partial results in float32 scratch (a slot per piece and head), merged by a second kernel
                piece_o = piece_ml = None
                if plan.n_cuts > 0:
                    rows = plan.n_pieces * hq * TILE_ROWS
                    piece_o = self._scratch("prefill pieces", rows * (hd + 2), torch.float32)
                    piece_ml = piece_o[rows * hd:]
                self._check(self.attn_tc.fz_attn_prefill_tc(
                    _p(q), c_int(n), _p(k), _p(v), c_longlong(page_stride), c_int(k.shape[0]), _p(meta.seg), _p(plan.tiles),
                    c_int(plan.n_tiles), _p(plan.cuts), c_int(plan.n_cuts), _p(piece_o), _p(piece_ml), _p(table),
                    c_int(table.shape[1]), c_int(cache.page_size), _p(out), c_int(hq),
                    c_int(hkv), c_int(hd), c_float(scale), c_int(window), _p(self.err), self._stream()),
                    "paged_attention (prefill, tcgen05)", kv_tiles)
                if plan.n_cuts > 0:
                    self.launches += 1    # the merge kernel
            elif plan.n_tiles > 0 and plan.n_cuts > 0:
                raise KernelError("paged_attention: the step's tiles are cut along the keys, which only the tcgen05 kernel takes")
            elif plan.n_tiles > 0:
                self._check(self.attn_tc.fz_attn_prefill(
                    _p(q), _p(k), _p(v), _p(meta.seg), _p(plan.tiles), c_int(plan.n_tiles), _p(table),
                    c_int(table.shape[1]), c_longlong(page_stride), c_int(cache.page_size), _p(out), c_int(hq),
                    c_int(hkv), c_int(hd), c_float(scale), c_int(window), self._stream()), "paged_attention (prefill)")
            return
        self._check(self.core.fz_attn_simt(
            _p(q), _p(k), _p(v), _p(meta.pos), _p(meta.seq_row), _p(table), c_int(table.shape[1]),
            c_longlong(page_stride), c_int(cache.page_size), _p(out), c_int(_CODE[self.dtype]), c_int(n), c_int(hq),
            c_int(hkv), c_int(hd), c_float(scale), c_int(window), _p(self.err), self._stream()), "paged_attention", kv)

    @staticmethod
    def _gate_kind(activation: str) -> int:
        kind = {"silu": 1, "gelu_tanh": 2}.get(activation)
        if kind is None:
            raise KernelError(f"gate activation {activation!r} is not one of 'silu', 'gelu_tanh'")
        return kind

    def swiglu(self, gate_up, out, activation: str = "silu") -> None:
        self._want(gate_up, "gate_up", (self.dtype,), 2)
        self._want(out, "swiglu output", (self.dtype,), 2)
        n, i = out.shape
        if gate_up.shape != (n, 2 * i):
            raise KernelError(f"swiglu: gate_up {tuple(gate_up.shape)}, out {tuple(out.shape)}")
        self._check(self.core.fz_swiglu(_p(gate_up), _p(out), c_int(_CODE[self.dtype]), c_int(n), c_int(i), c_int(self._gate_kind(activation)),
                                        self._stream()), "swiglu")

    def argmax(self, logits, out) -> None:
        self._want(logits, "logits", (torch.float32,), 2)
        self._want(out, "argmax output", (torch.int32,), 1)
        r, v = logits.shape
        if out.shape[0] != r:
            raise KernelError(f"argmax: logits {tuple(logits.shape)}, out {tuple(out.shape)}")
        # scratch of the row-split argmax: per row up to S partial (value, index) pairs and one counter (kept zero)
        cap, slices = max(r, 64), int(self.core.fz_argmax_max_slices())
        pv = self._scratch("argmax partial values", cap * slices, torch.float32)
        pi = self._scratch("argmax partial indices", cap * slices, torch.int32)
        cnt = self._scratch("argmax counters", cap, torch.int32, zero=True)
        self._check(self.core.fz_argmax(_p(logits), _p(out), c_int(r), c_int(v), _p(pv), _p(pi), _p(cnt), self._stream()),
                    "argmax")

    def sample(self, logits, temperature, uniform, out) -> None:
        self._want(logits, "logits", (torch.float32,), 2)
        self._want(temperature, "temperature", (torch.float32,), 1)
        self._want(uniform, "uniform", (torch.float64,), 1)
        self._want(out, "sample output", (torch.int32,), 1)
        r, v = logits.shape
        if out.shape[0] != r or temperature.shape[0] != r or uniform.shape[0] != r:
            raise KernelError("sample: row counts differ")
        self._check(self.core.fz_sample(_p(logits), _p(temperature), _p(uniform), _p(out), c_int(r), c_int(v),
                                        self._stream()), "sample")

    def sample_filtered(self, logits, temperature, top_k, top_p, uniform, out) -> None:
        self._want(logits, "logits", (torch.float32,), 2)
        self._want(temperature, "temperature", (torch.float32,), 1)
        self._want(top_k, "top_k", (torch.int32,), 1)
        self._want(top_p, "top_p", (torch.float32,), 1)
        self._want(uniform, "uniform", (torch.float64,), 1)
        self._want(out, "sample output", (torch.int32,), 1)
        r, v = logits.shape
        if any(t.shape[0] != r for t in (out, temperature, top_k, top_p, uniform)):
            raise KernelError("sample_filtered: row counts differ")
        weights = self._scratch("sampling weights", r * v, torch.float64)       # exp(x / T - max) of every token
        self._check(self.core.fz_sample_filtered(_p(logits), _p(temperature), _p(top_k), _p(top_p), _p(uniform), _p(weights),
                                                 _p(out), c_int(r), c_int(v), self._stream()), "sample_filtered")

    # ---- the gated parallel block
    def select_tokens(self, tokens, src, prev_ids, out) -> None:
        for t, name in ((tokens, "tokens"), (src, "src"), (prev_ids, "prev_ids"), (out, "token ids")):
            self._want(t, name, (torch.int32,), 1)
        n = tokens.shape[0]
        if src.shape[0] != n or out.shape[0] != n:
            raise KernelError("select_tokens: row counts differ")
        self._check(self.mix.fz_select_tokens(_p(tokens), _p(src), _p(prev_ids), _p(out), c_int(n), self._stream()), "select_tokens")

    def short_conv(self, h, w, state, meta, out, residual: bool = True, activation: str | None = None, bias=None) -> None:
        if activation not in (None, "silu"):
            raise KernelError(f"short_conv: activation {activation!r} is not one of None, 'silu'")
        self._want(h, "convolution input", (self.dtype,), 2)
        self._want(w, "convolution weight", (self.dtype,), 2)
        self._want(out, "convolution output", (self.dtype,), 2)
        n, c = h.shape
        taps = w.shape[1]
        if bias is not None:
            self._want(bias, "convolution bias", (torch.float32,), 1)
            if bias.shape[0] != c:
                raise KernelError(f"short_conv: bias {tuple(bias.shape)} for {c} channels")
        if w.shape[0] != c or out.shape != h.shape:
            raise KernelError(f"short_conv: h {tuple(h.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
        if taps > 1:
            if state is None:
                raise KernelError("short_conv: a convolution of more than one tap needs its state")
            self._want(state, "convolution state", (torch.float32,), 3)
            if tuple(state.shape[1:]) != (taps - 1, c):
                raise KernelError(f"short_conv: state {tuple(state.shape)}, expected (slots, {taps - 1}, {c})")
        self._check(self.mix.fz_short_conv(_p(h), _p(w), _p(state), _p(meta.seg), _p(meta.seq_row), _p(out),
                                           c_int(_CODE[self.dtype]), c_int(n), c_int(getattr(meta, "max_segments", meta.n_segments)), c_int(c), c_int(taps),
                                           c_int(1 if residual else 0), c_int(1 if activation else 0), _p(bias), self._stream()), "short_conv",
                    n * c * 2 * h.element_size())
        if taps > 1:
            self.launches += 1    # the state update

    def gated_sum(self, a, gate_a, f, gate_f, out, f_terms: int = 1, f_weight: float = 1.0) -> None:
        n, d = a.shape
        for t, name, rows in ((a, "a", n), (gate_a, "gate_a", n), (f, "f", n * f_terms), (gate_f, "gate_f", n), (out, "out", n)):
            if t is not None:
                self._want(t, name, (torch.float32,), 2)
                if tuple(t.shape) != (rows, d):
                    raise KernelError(f"gated_sum: {name} {tuple(t.shape)}, expected {(rows, d)}")
        self._check(self.mix.fz_gated_sum(_p(a), _p(gate_a), _p(f), _p(gate_f), _p(out), c_int(n), c_int(d), c_int(f_terms),
                                          c_float(f_weight), self._stream()), "gated_sum",
                    n * d * 4 * (2 + (gate_a is not None) + (gate_f is not None) + (f_terms if f is not None else 0)))

    def scale_(self, x, factor: float) -> None:
        self._want(x, "x", (torch.float32,))
        self._check(self.mix.fz_scale(_p(x), c_float(factor), c_longlong(x.numel()), self._stream()), "scale")

    # ---- latent attention
    def check_latent_attention(self, num_heads: int, key_width: int, value_width: int) -> None:
        if self.latent.fz_attn_latent_check(c_int(num_heads), c_int(key_width), c_int(value_width)) != 0:
            raise ValueError(f"latent attention sizes not supported: {num_heads} heads, cached vectors of {key_width} "
                             f"values of which {value_width} are read as values (need value <= key <= 1024, value <= 512)")
        if self.use_tensor_cores and self.latent_tensor_cores:
            self.latent_tc    # built and loaded with the model, not at its first step

    def _latent_pool(self, cache, width: int):
        pool = cache.keys
        if not pool.is_cuda or pool.dtype != self.dtype:
            raise KernelError(f"latent pool: device {pool.device}, dtype {pool.dtype}; expected CUDA {self.dtype}")
        if pool.dim() != 3 or pool.shape[1] != cache.page_size or pool.shape[2] != width or pool.stride(2) != 1 \
                or pool.stride(1) != width:
            raise KernelError(f"latent pool has shape {tuple(pool.shape)} and strides {pool.stride()}, expected "
                              f"(pages, {cache.page_size}, {width}) with contiguous pages")
        return pool, pool.stride(0)

    def latent_cache_write(self, down, norm_weight, eps, cos, sin, rotated, meta, cache, pairing: int = 0) -> None:
        self._want(down, "latent projection", (torch.float32,), 2)
        self._want(norm_weight, "latent norm weight", (torch.float32, torch.bfloat16), 1)
        self._want(cos, "cos table", (torch.float32,), 2)
        self._want(sin, "sin table", (torch.float32,), 2)
        n, width = down.shape
        lat = norm_weight.shape[0]
        rot = width - lat
        if rot < 0 or rotated > rot or rotated % 2 or cos.shape[1] != rotated // 2 or sin.shape != cos.shape:
            raise KernelError(f"latent_cache_write: down {tuple(down.shape)}, latent {lat}, rotated {rotated}, cos {tuple(cos.shape)}")
        pool, page_stride = self._latent_pool(cache, width)
        table = meta.table(cache.group)
        self._check(self.mix.fz_latent_cache_write(
            _p(down), _p(norm_weight), c_int(_CODE[norm_weight.dtype]), c_float(eps), _p(cos), _p(sin), c_int(rotated),
            _p(meta.pos), _p(meta.seq_row), _p(table), c_int(table.shape[1]), _p(pool), c_int(_CODE[self.dtype]),
            c_longlong(page_stride), c_int(cache.page_size), c_int(n), c_int(lat), c_int(rot), c_int(cos.shape[0]),
            c_int(pool.shape[0]), c_int(pairing), _p(self.err), self._stream()), "latent_cache_write",
            n * width * (4 + pool.element_size()))

    def rotate_heads(self, q, offset, cos, sin, rotated, meta, out, out_offset, pairing: int = 0) -> None:
        self._want(q, "q", (self.dtype,), 3)
        self._want(out, "rotated q", (self.dtype,), 3)
        self._want(cos, "cos table", (torch.float32,), 2)
        self._want(sin, "sin table", (torch.float32,), 2)
        n, heads, w = q.shape
        if out.shape[:2] != q.shape[:2] or out_offset + w - offset > out.shape[2] or cos.shape[1] != rotated // 2 \
                or sin.shape != cos.shape or rotated > w - offset:
            raise KernelError(f"rotate_heads: q {tuple(q.shape)} from {offset}, out {tuple(out.shape)} at {out_offset}, rotated {rotated}")
        self._check(self.mix.fz_rotate_heads(_p(q), c_int(w), c_int(offset), _p(cos), _p(sin), c_int(rotated), _p(meta.pos),
                                             _p(meta.seq_row), _p(out), c_int(out.shape[2]), c_int(out_offset),
                                             c_int(_CODE[self.dtype]), c_int(n), c_int(heads), c_int(cos.shape[0]),
                                             c_int(pairing), _p(self.err), self._stream()), "rotate_heads")

    def linear_heads(self, a, a_offset, k, w, out, out_offset) -> None:
        self._want(a, "per-head input", (self.dtype,), 3)
        self._want(w, "per-head weight", (self.dtype,), 3)
        self._want(out, "per-head output", (self.dtype, torch.float32), 3)
        n, heads, wa = a.shape
        m = w.shape[1]
        if w.shape[0] != heads or w.shape[2] != k or a_offset + k > wa or out.shape[:2] != a.shape[:2] \
                or out_offset + m > out.shape[2]:
            raise KernelError(f"linear_heads: a {tuple(a.shape)} from {a_offset}, w {tuple(w.shape)}, out {tuple(out.shape)} at {out_offset}")
        es, eo = a.element_size(), out.element_size()
        if self.use_tensor_cores and self.grouped_tensor_cores:
            args = (c_void_p(a.data_ptr() + a_offset * es), c_longlong(heads * wa), c_longlong(wa), _p(w),
                    c_void_p(out.data_ptr() + out_offset * eo), c_longlong(heads * out.shape[2]), c_longlong(out.shape[2]))
            if self.mix_tc.fz_grouped_tc_check(*args, c_int(m), c_int(k)) == 0:
                self._check(self.mix_tc.fz_linear_heads_tc(*args, c_int(_CODE[out.dtype]), c_int(n), c_int(heads), c_int(m),
                                                           c_int(k), self._stream()), "linear_heads (tensor cores)",
                            (n * heads * (k + m) + heads * m * k) * es)
                return
        self._check(self.mix.fz_linear_heads(
            c_void_p(a.data_ptr() + a_offset * es), c_longlong(heads * wa), c_longlong(wa), _p(w),
            c_void_p(out.data_ptr() + out_offset * eo), c_longlong(heads * out.shape[2]), c_longlong(out.shape[2]),
            c_int(_CODE[self.dtype]), c_int(_CODE[out.dtype]), c_int(n), c_int(heads), c_int(m), c_int(k), self._stream()),
            "linear_heads", (n * heads * (k + m) + heads * m * k) * es)

    def latent_attention(self, q, cache, meta, out, value_width, scale, window, sink=None) -> None:
        self._want(q, "q", (self.dtype,), 3)
        if sink is not None:
            self._want(sink, "sinks", (torch.float32,), 1)
            if sink.shape[0] != q.shape[1]:
                raise KernelError(f"latent_attention: {tuple(sink.shape)} sinks for {q.shape[1]} heads")
        self._want(out, "attention output", (self.dtype,), 3)
        n, heads, width = q.shape
        if tuple(out.shape) != (n, heads, value_width):
            raise KernelError(f"latent_attention: q {tuple(q.shape)}, out {tuple(out.shape)}, values {value_width}")
        pool, page_stride = self._latent_pool(cache, width)
        table = meta.table(cache.group)
        nbytes = 0
        if self._profile is not None:
            nbytes = contexts(list(getattr(meta, "segments", ()))) * width * pool.element_size() + n * heads * (width + value_width) * q.element_size()
        if self.use_tensor_cores and self.latent_tensor_cores and \
                self.latent_tc.fz_attn_latent_tc_check(c_int(heads), c_int(width), c_int(value_width)) == 0:
            blocks = n * heads // 64 + max(1, int(getattr(meta, "latent_extra", 0)) or n)
            # few tiles with many keys behind them (decoded tokens): the keys are cut into ranges, merged by a second kernel
            ctx = max(1, int(meta.max_context))
            splits = int(self.latent_tc.fz_attn_latent_tc_splits(c_int(blocks), c_int(ctx), c_int(self._sms))) if self.latent_key_cuts else 1
            scratch = None
            if splits > 1:
                self.latent_tc.fz_attn_latent_tc_scratch.restype = c_longlong
                scratch = self._scratch("latent attention partials",
                                        int(self.latent_tc.fz_attn_latent_tc_scratch(c_int(blocks), c_int(splits), c_int(value_width))),
                                        torch.float32)
            self._check(self.latent_tc.fz_attn_latent_tc(
                _p(q), _p(pool), _p(meta.seq_row), _p(meta.seg), c_int(meta.n_segments), _p(table), c_int(table.shape[1]),
                c_longlong(page_stride), c_int(cache.page_size), c_int(pool.shape[0]), _p(out), c_int(n), c_int(blocks),
                c_int(heads), c_int(width), c_int(value_width), c_float(scale), c_int(window), c_int(splits), c_int(ctx),
                _p(scratch), _p(sink), _p(self.err), self._stream()),
                "latent_attention (tensor cores)", nbytes)
            self.launches += 2 if splits > 1 else 1    # the kernel that zeroes rows of padding, the merge kernel
            return
        self._check(self.latent.fz_attn_latent(
            _p(q), _p(pool), _p(meta.pos), _p(meta.seq_row), _p(table), c_int(table.shape[1]), c_longlong(page_stride),
            c_int(cache.page_size), c_int(pool.shape[0]), _p(out), c_int(_CODE[self.dtype]), c_int(n), c_int(heads),
            c_int(width), c_int(value_width), c_float(scale), c_int(window), _p(sink), _p(self.err), self._stream()),
            "latent_attention", nbytes)

    # ---- experts chosen by a table
    def route_by_table(self, token_ids, meta, table, num_experts, align: int = 1):
        self._want(token_ids, "token ids", (torch.int32,), 1)
        self._want(table, "expert table", (torch.int32,), 2)
        return self._sort_pairs(token_ids, token_ids.shape[0], meta, table, num_experts, align)

    def _sort_pairs(self, token_ids, n, meta, table, num_experts, align):
        """The step's (row, choice) pairs sorted by expert table[id of the row, choice] (no ids: table[row, choice])."""
        top = table.shape[1]
        # row tiles of 64 pairs; of 16 where an expert gets few rows (decoded tokens) and the tensor-core kernels run
        tile = int(self.mix.fz_grouped_tile_rows())
        if self.use_tensor_cores and self.grouped_tensor_cores and n * top <= 16 * num_experts:
            tile = 16
        elif self.grouped_tiles_128 and self.use_tensor_cores and self.grouped_tensor_cores and align % 8 == 0 \
                and n * top >= 192 * num_experts:
            tile = 128      # (only where the sizes are sure to go to the tensor-core kernels: the plain ones take 64 at most)
        max_tiles = -(-n * top // tile) + min(num_experts, n * top)
        idx = self._scratch("expert route", 2 * n * top + 3 * max_tiles, torch.int32)
        a_idx, c_idx, tiles = idx[:n * top], idx[n * top: 2 * n * top], idx[2 * n * top: 2 * n * top + 3 * max_tiles]
        self._check(self.mix.fz_route_by_table(_p(token_ids), _p(meta.seq_row), _p(table), c_int(n), c_int(table.shape[0]),
                                               c_int(top), c_int(num_experts), _p(a_idx), _p(c_idx), _p(tiles),
                                               c_int(max_tiles), c_int(tile), _p(self.err), self._stream()), "route_by_table")
        return (a_idx, c_idx, tiles, max_tiles, n, top, meta.seq_row, tile)

    def _grouped_tc(self, a, lda, w, c, ldc, n_out, k) -> bool:
        return bool(self.use_tensor_cores and self.grouped_tensor_cores and a.dtype == torch.bfloat16 and
                    self.mix_tc.fz_grouped_tc_check(_p(a), c_longlong(lda), c_longlong(0), _p(w), _p(c), c_longlong(ldc),
                                                    c_longlong(0), c_int(n_out), c_int(k)) == 0)

    def grouped_linear_glu(self, h, w, route, y, alpha, limit, up_shift: float = 1.0) -> None:
        a_idx, c_idx, tiles, max_tiles, n, top, seq_row, tile = route
        self._want(h, "expert input", (self.dtype,), 2)
        self._want(w, "expert gate/up weights", (self.dtype,), 3)
        self._want(y, "expert activation", (self.dtype,), 2)
        k, inter = h.shape[1], w.shape[1] // 2
        if h.shape[0] != n or w.shape[2] != k or w.shape[1] != 2 * inter or tuple(y.shape) != (n * top, inter):
            raise KernelError(f"grouped_linear_glu: h {tuple(h.shape)}, w {tuple(w.shape)}, y {tuple(y.shape)}")
        nbytes = (min(w.shape[0], n * top) * 2 * inter * k + n * k + n * top * inter) * h.element_size()
        if self._grouped_tc(h, k, w, y, inter, inter, k):
            self._check(self.mix_tc.fz_grouped_linear_tc(_p(h), _p(w), _p(y), _p(tiles), c_int(max_tiles), c_int(tile), _p(a_idx),
                                                         c_void_p(0), c_int(_CODE[y.dtype]), c_int(inter), c_int(k), c_int(1),
                                                         c_float(alpha), c_float(limit), c_float(up_shift), c_void_p(0), c_int(0), c_int(0),
                                                         self._stream()), "grouped_linear_glu (tensor cores)", nbytes)
            return
        self._check(self.mix.fz_grouped_linear(_p(h), _p(w), _p(y), _p(tiles), c_int(max_tiles), c_int(tile), _p(a_idx), c_void_p(0),
                                               c_int(_CODE[self.dtype]), c_int(_CODE[self.dtype]), c_int(inter), c_int(k),
                                               c_int(1), c_float(alpha), c_float(limit), c_float(up_shift), c_void_p(0), c_int(0), c_int(0),
                                               self._stream()),
                    "grouped_linear_glu", (min(w.shape[0], n * top) * 2 * inter * k + n * k + n * top * inter) * h.element_size())

    def grouped_linear_scatter(self, y, w, route, out) -> None:
        a_idx, c_idx, tiles, max_tiles, n, top, seq_row, tile = route
        self._want(y, "expert activation", (self.dtype,), 2)
        self._want(w, "expert down weights", (self.dtype,), 3)
        self._want(out, "expert outputs", (torch.float32,), 2)
        inter, d = y.shape[1], w.shape[1]
        if y.shape[0] != n * top or w.shape[2] != inter or tuple(out.shape) != (n * top, d):
            raise KernelError(f"grouped_linear_scatter: y {tuple(y.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
        nbytes = min(w.shape[0], n * top) * d * inter * y.element_size() + n * top * (inter * y.element_size() + d * 4)
        if self._grouped_tc(y, inter, w, out, d, d, inter):
            self._check(self.mix_tc.fz_grouped_linear_tc(_p(y), _p(w), _p(out), _p(tiles), c_int(max_tiles), c_int(tile),
                                                         c_void_p(0), _p(c_idx), c_int(_CODE[out.dtype]), c_int(d), c_int(inter),
                                                         c_int(0), c_float(0.0), c_float(0.0), c_float(0.0), _p(seq_row), c_int(n), c_int(top),
                                                         self._stream()), "grouped_linear_scatter (tensor cores)", nbytes)
            return
        self._check(self.mix.fz_grouped_linear(_p(y), _p(w), _p(out), _p(tiles), c_int(max_tiles), c_int(tile), c_void_p(0), _p(c_idx),
                                               c_int(_CODE[self.dtype]), c_int(_CODE[torch.float32]), c_int(d), c_int(inter),
                                               c_int(0), c_float(0.0), c_float(0.0), c_float(0.0), _p(seq_row), c_int(n), c_int(top),
                                               self._stream()),
                    "grouped_linear_scatter", min(w.shape[0], n * top) * d * inter * y.element_size() + n * top * (inter * y.element_size() + d * 4))

    # ---- recurrent mixers, attention with a window, kept first tokens and a sink, routed experts
    def recurrent_state_shape(self, heads: int, key_dim: int, value_dim: int) -> tuple:
        """(heads, value_dim, padded key_dim): a column of S is contiguous, padded to 8 times a power of two."""
        pad = int(self.seq.fz_recurrent_key_pad(c_int(key_dim)))
        if pad < 0:
            raise ValueError(f"a recurrent state with {key_dim} key dimensions is not supported (1..256)")
        return (heads, value_dim, pad)

    def _state(self, state, heads, key_dim, value_dim, what):
        self._want(state, f"{what} state", (torch.float32,), 4)
        if tuple(state.shape[1:]) != self.recurrent_state_shape(heads, key_dim, value_dim):
            raise KernelError(f"{what}: state {tuple(state.shape)}, expected (slots, "
                              f"{', '.join(map(str, self.recurrent_state_shape(heads, key_dim, value_dim)))})")

    def _tables(self, cos, sin, rotated, what):
        if not rotated:
            return 0
        self._want(cos, "cos table", (torch.float32,), 2)
        self._want(sin, "sin table", (torch.float32,), 2)
        if rotated % 2 or cos.shape[1] != rotated // 2 or sin.shape != cos.shape:
            raise KernelError(f"{what}: {rotated} rotated dimensions, cos {tuple(cos.shape)}, sin {tuple(sin.shape)}")
        return cos.shape[0]

    def retention_scan(self, proj, heads, key_dim, value_dim, decay, key_scale, cos, sin, rotated, pairing, state, meta, out) -> None:
        self._want(proj, "retention projections", (torch.float32,), 2)
        self._want(decay, "decay", (torch.float32,), 1)
        self._want(out, "retention output", (torch.float32,), 2)
        n, ld = proj.shape
        if ld < heads * (2 * key_dim + value_dim) or tuple(out.shape) != (n, heads * value_dim) or decay.shape[0] != heads:
            raise KernelError(f"retention_scan: proj {tuple(proj.shape)}, out {tuple(out.shape)}, decay {tuple(decay.shape)}")
        self._state(state, heads, key_dim, value_dim, "retention_scan")
        self._meta_rows = meta.seq_row
        max_pos = self._tables(cos, sin, rotated, "retention_scan")
        self._check(self.seq.fz_retention_scan(
            _p(proj), c_int(ld), c_int(heads), c_int(key_dim), c_int(value_dim), _p(decay), c_float(key_scale),
            _p(cos if rotated else None), _p(sin if rotated else None), c_int(rotated), c_int(pairing), c_int(max_pos), _p(state),
            _p(meta.seg), c_int(meta.max_segments), _p(out), _p(self.err), self._stream()), "retention_scan",
            n * heads * (2 * key_dim + 2 * value_dim) * 4 + 2 * meta.n_segments * heads * value_dim * state.shape[3] * 4)

    def gated_delta_scan(self, qkv, heads, key_heads, key_dim, value_dim, high, beta, a_log, dt_bias, unit_eps, query_scale,
                         state, meta, out) -> None:
        self._want(qkv, "q/k/v", (self.dtype,), 2)
        self._want(high, "decay inputs", (torch.float32,), 2)
        self._want(beta, "beta", (torch.float32,), 2)
        self._want(a_log, "decay rates", (torch.float32,), 1)
        self._want(dt_bias, "decay bias", (torch.float32,), 1)
        self._want(out, "delta-rule output", (torch.float32,), 2)
        n = qkv.shape[0]
        if qkv.shape[1] != 2 * key_heads * key_dim + heads * value_dim or high.shape[0] != n or high.shape[1] < heads * key_dim \
                or tuple(beta.shape) != (n, heads) or a_log.shape[0] != heads or dt_bias.shape[0] != heads * key_dim \
                or tuple(out.shape) != (n, heads * value_dim) or heads % key_heads:
            raise KernelError(f"gated_delta_scan: qkv {tuple(qkv.shape)}, high {tuple(high.shape)}, beta {tuple(beta.shape)}, "
                              f"out {tuple(out.shape)}")
        self._state(state, heads, key_dim, value_dim, "gated_delta_scan")
        self._meta_rows = meta.seq_row
        self._check(self.seq.fz_gated_delta_scan(
            _p(qkv), c_int(_CODE[self.dtype]), c_int(heads), c_int(key_heads), c_int(key_dim), c_int(value_dim), _p(high),
            c_int(high.shape[1]), _p(beta), _p(a_log), _p(dt_bias), c_float(unit_eps), c_float(query_scale), _p(state),
            _p(meta.seg), c_int(meta.max_segments), _p(out), self._stream()), "gated_delta_scan",
            n * (qkv.shape[1] * qkv.element_size() + heads * (key_dim + value_dim + 1) * 4)
            + 2 * meta.n_segments * heads * value_dim * state.shape[3] * 4)

    def head_norm_gate(self, o, heads, value_dim, weight, eps, gate, gate_offset, activation, out) -> None:
        self._want(o, "head outputs", (torch.float32,), 2)
        self._want(out, "normed head outputs", (torch.float32, self.dtype), 2)
        n = o.shape[0]
        if o.shape[1] != heads * value_dim or out.shape != o.shape:
            raise KernelError(f"head_norm_gate: o {tuple(o.shape)}, out {tuple(out.shape)}, {heads} heads of {value_dim}")
        if weight is not None:
            self._want(weight, "head norm weight", (torch.float32,), 1)
            if weight.shape[0] not in (value_dim, heads * value_dim):
                raise KernelError(f"head_norm_gate: weight {tuple(weight.shape)} for {heads} heads of {value_dim}")
        act = {None: 0, "sigmoid": 1, "silu": 2}.get(activation, -1)
        if act < 0:
            raise KernelError(f"head_norm_gate: activation {activation!r} is not one of None, 'sigmoid', 'silu'")
        ldg = 0
        if gate is not None:
            self._want(gate, "gate", (torch.float32,), 2)
            ldg = gate.shape[1]
            if gate.shape[0] != n or gate_offset + heads * value_dim > ldg or act == 0:
                raise KernelError(f"head_norm_gate: gate {tuple(gate.shape)} from column {gate_offset}, activation {activation!r}")
        seq_row = self._step_rows(n)
        per_head = 1 if weight is not None and heads > 1 and weight.shape[0] == heads * value_dim else 0
        self._check(self.seq.fz_head_norm_gate(_p(o), c_int(n), c_int(heads), c_int(value_dim), _p(weight), c_int(per_head), c_float(eps),
                                               _p(gate), c_int(ldg), c_int(gate_offset), c_int(act if gate is not None else 0),
                                               _p(seq_row), _p(out), c_int(_CODE[out.dtype]), self._stream()),
                    "head_norm_gate", n * heads * value_dim * (4 + (4 if gate is not None else 0) + out.element_size()))

    def _step_rows(self, n: int):
        """meta.seq_row of the step being run (the ops that take no `meta` still zero their rows of padding)."""
        rows = self._meta_rows
        if rows is None or rows.shape[0] != n:
            raise KernelError("the step's rows are not known: `route_by_scores`, `rotate_kv_write` or a scan must run first")
        return rows

    def check_sink_attention(self, num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int) -> None:
        if self.seq.fz_sink_attention_check(c_int(num_heads), c_int(num_kv_heads), c_int(key_dim), c_int(value_dim)) != 0:
            raise ValueError(f"attention sizes not supported: {num_heads} heads, {num_kv_heads} kv heads, key size {key_dim}, "
                             f"value size {value_dim} (need heads % kv_heads == 0 and sizes of 1..512)")
        if self.use_tensor_cores and self.sink_tensor_cores and key_dim == value_dim and key_dim in (64, 128):
            self.seq_tc       # built and loaded with the model, not at its first step

    def _kv_views(self, cache, hkv: int, dk: int, dv: int):
        k, v = cache.keys, cache.values
        for t, name, d in ((k, "key pool", dk), (v, "value pool", dv)):
            if not t.is_cuda or t.dtype != self.dtype:
                raise KernelError(f"{name}: device {t.device}, dtype {t.dtype}; expected CUDA {self.dtype}")
            if t.dim() != 4 or t.shape[1] != hkv or t.shape[2] != cache.page_size or t.shape[3] != d or t.stride(3) != 1:
                raise KernelError(f"{name} has shape {tuple(t.shape)} and strides {t.stride()}, expected (pages, {hkv}, "
                                  f"{cache.page_size}, {d}) with a unit last stride")
        if k.stride()[:3] != v.stride()[:3]:
            raise KernelError("key and value pools have different strides")
        return k, v

    def rotate_kv_write(self, qkv, cos, sin, rotated, pairing, meta, cache, q_out, num_heads, num_kv_heads, key_dim, value_dim,
                        q_norm=None, k_norm=None, norm_eps: float = 0.0, query_temperature=None) -> None:
        self._want(qkv, "qkv", (torch.float32,), 2)
        self._want(q_out, "q", (self.dtype,), 2)
        n = qkv.shape[0]
        need = (num_heads + num_kv_heads) * key_dim + num_kv_heads * value_dim if cache.write else num_heads * key_dim
        if qkv.shape[1] < need or tuple(q_out.shape) != (n, num_heads * key_dim):
            raise KernelError(f"rotate_kv_write: qkv {tuple(qkv.shape)}, q {tuple(q_out.shape)}")
        for w, name in ((q_norm, "q norm weight"), (k_norm, "k norm weight")):
            if w is not None:
                self._want(w, name, (torch.float32,), 1)
                if w.shape[0] != key_dim:
                    raise KernelError(f"rotate_kv_write: {name} {tuple(w.shape)} for heads of {key_dim}")
        if cache.write and (q_norm is None) != (k_norm is None):
            raise KernelError("rotate_kv_write: queries and keys are normed together or not at all")
        coef, every = (float(query_temperature[0]), int(query_temperature[1])) if query_temperature is not None else (0.0, 0)
        self._meta_rows = meta.seq_row
        max_pos = self._tables(cos, sin, rotated, "rotate_kv_write")
        k, v = self._kv_views(cache, num_kv_heads, key_dim, value_dim)
        table = meta.table(cache.group)
        self._check(self.seq.fz_rotate_kv_write(
            _p(qkv), c_int(qkv.shape[1]), _p(cos if rotated else None), _p(sin if rotated else None), c_int(rotated), c_int(pairing), c_int(max_pos),
            _p(meta.pos), _p(meta.seq_row), _p(table), c_int(table.shape[1]), _p(k), _p(v), c_longlong(k.stride(0)),
            c_longlong(k.stride(1)), c_longlong(k.stride(2)), c_int(cache.page_size), c_int(k.shape[0]),
            c_int(1 if cache.write else 0), _p(q_out), c_int(_CODE[self.dtype]), c_int(n), c_int(num_heads), c_int(num_kv_heads),
            c_int(key_dim), c_int(value_dim), _p(q_norm), _p(k_norm), c_float(norm_eps), c_float(coef), c_int(every),
            _p(self.err), self._stream()), "rotate_kv_write", n * need * (4 + q_out.element_size()))

    def sink_attention(self, q, cache, meta, out, num_heads, num_kv_heads, key_dim, value_dim, scale, window, keep_first, sink,
                       softcap: float = 0.0, gate=None, span: int = 0) -> None:
        self._want(q, "q", (self.dtype,), 2)
        self._want(out, "attention output", (self.dtype,), 2)
        n = q.shape[0]
        if q.shape[1] != num_heads * key_dim or tuple(out.shape) != (n, num_heads * value_dim):
            raise KernelError(f"sink_attention: q {tuple(q.shape)}, out {tuple(out.shape)}")
        if span < 0 or (span and keep_first):
            raise KernelError(f"sink_attention: a chunked mask of {span} positions with {keep_first} kept first tokens")
        if sink is not None:
            self._want(sink, "sinks", (torch.float32,), 1)
            if sink.shape[0] != num_heads:
                raise KernelError(f"sink_attention: {tuple(sink.shape)} sinks for {num_heads} heads")
        g, g_off, g_ld = None, 0, 0
        if gate is not None:
            g, g_off = gate
            self._want(g, "head gates", (torch.float32,), 2)
            g_ld = g.shape[1]
            if g.shape[0] != n or g_off < 0 or g_off + num_heads > g_ld:
                raise KernelError(f"sink_attention: gates {tuple(g.shape)} from column {g_off} for {num_heads} heads")
        k, v = self._kv_views(cache, num_kv_heads, key_dim, value_dim)
        table = meta.table(cache.group)
        nbytes = 0
        if self._profile is not None:
            seen = sum(min(sg.pos0 + i + 1, (window + keep_first) if window else sg.pos0 + i + 1, (sg.pos0 + i) % span + 1 if span else 1 << 62)
                       for sg in meta.segments for i in range(sg.n))
            nbytes = seen * num_kv_heads * (key_dim + value_dim) * k.element_size() + n * num_heads * (key_dim + value_dim) * q.element_size()
        # A step of single tokens (bfloat16): a row's keys are cut into runs of chunks, one block each, and merged by a
        # second kernel, so that a few rows fill the GPU. Other steps: blocks of consecutive rows of a portion that share
        # their key and value loads. (float32 keeps the one arithmetic for every step: a position's bits do not depend
        # on the cutting.)
        max_portion = max(1, int(getattr(meta, "max_portion", 0)) or n)
        n_seg = getattr(meta, "max_segments", meta.n_segments)
        # prompt portions (bfloat16, keys and values of size 64 or 128): tiles of 64 rows on tensor cores
        if self.use_tensor_cores and self.sink_tensor_cores and self.dtype == torch.bfloat16 and max_portion >= SINK_MMA_ROWS and \
                key_dim == value_dim and key_dim in (64, 128) and self.seq_tc.fz_sink_attention_mma_check(
                    c_int(num_heads), c_int(num_kv_heads), c_int(key_dim), c_int(value_dim), _p(k), _p(v), c_longlong(k.stride(0)),
                    c_longlong(k.stride(1)), c_longlong(k.stride(2))) == 0:
            self._check(self.seq_tc.fz_sink_attention_mma(
                _p(q), _p(k), _p(v), _p(meta.seg), _p(meta.seq_row), c_int(n_seg), c_int(max_portion), _p(table),
                c_int(table.shape[1]), c_longlong(k.stride(0)), c_longlong(k.stride(1)), c_longlong(k.stride(2)),
                c_int(cache.page_size), c_int(k.shape[0]), _p(out), c_int(n), c_int(num_heads), c_int(num_kv_heads),
                c_int(key_dim), c_float(scale), c_int(window), c_int(keep_first), _p(sink), c_float(softcap), _p(g), c_int(g_ld),
                c_int(g_off), c_int(span), _p(self.err), self._stream()), "sink_attention (tensor cores)", nbytes)
            return
        unit_chunks = units = 0
        part = None
        if self.split_decode_keys and self.dtype == torch.bfloat16 and max_portion == 1:
            ctx = max(1, int(meta.max_context))
            reach = min(window or ctx, span or ctx)      # the most keys a row sees, kept first tokens aside
            unit_chunks = 2 if window else max(2, -(-reach // (32 * self.sink_max_runs)))
            units = int(self.seq.fz_sink_attention_units(c_int(window), c_int(keep_first), c_int(ctx), c_int(unit_chunks), c_int(span)))
            part = self._scratch("sink attention partials", n * num_heads * units * (value_dim + 2), torch.float32)
        self._check(self.seq.fz_sink_attention(
            _p(q), _p(k), _p(v), _p(meta.pos), _p(meta.seq_row), _p(meta.seg), c_int(getattr(meta, "max_segments", meta.n_segments)),
            c_int(max_portion), _p(table), c_int(table.shape[1]), c_longlong(k.stride(0)),
            c_longlong(k.stride(1)), c_longlong(k.stride(2)), c_int(cache.page_size), c_int(k.shape[0]), _p(out),
            c_int(_CODE[self.dtype]), c_int(n), c_int(num_heads), c_int(num_kv_heads), c_int(key_dim), c_int(value_dim),
            c_float(scale), c_int(window), c_int(keep_first), _p(sink), c_int(unit_chunks), c_int(units), _p(part),
            c_float(softcap), _p(g), c_int(g_ld), c_int(g_off), c_int(span), _p(self.err), self._stream()), "sink_attention", nbytes)
        if units:
            self.launches += 1      # the merge kernel

    def general_delta_scan(self, proj, heads, key_dim, value_dim, remove_offset, decay_in, decay_bias, remove_bias, decay_rate,
                           unit_eps, state, meta, out) -> None:
        self._want(proj, "delta-rule projections", (torch.float32,), 2)
        self._want(decay_in, "decay inputs", (torch.float32,), 2)
        self._want(decay_bias, "decay bias", (torch.float32,), 1)
        self._want(remove_bias, "removal bias", (torch.float32,), 1)
        self._want(out, "delta-rule output", (torch.float32,), 2)
        n, ld = proj.shape
        hk = heads * key_dim
        if ld < 2 * hk + heads * value_dim or not 0 <= remove_offset <= ld - hk or tuple(decay_in.shape) != (n, hk) or \
                decay_bias.shape[0] != hk or remove_bias.shape[0] != hk or tuple(out.shape) != (n, heads * value_dim):
            raise KernelError(f"general_delta_scan: proj {tuple(proj.shape)}, decay inputs {tuple(decay_in.shape)}, "
                              f"out {tuple(out.shape)}, removal inputs from column {remove_offset}")
        self._state(state, heads, key_dim, value_dim, "general_delta_scan")
        self._meta_rows = meta.seq_row
        self._check(self.seq.fz_general_delta_scan(
            _p(proj), c_int(ld), c_int(heads), c_int(key_dim), c_int(value_dim), c_int(remove_offset), _p(decay_in),
            _p(decay_bias), _p(remove_bias), c_float(decay_rate), c_float(unit_eps), _p(state), _p(meta.seg),
            c_int(meta.max_segments), _p(out), self._stream()), "general_delta_scan",
            n * heads * (4 * key_dim + 2 * value_dim) * 4 + 2 * meta.n_segments * heads * value_dim * state.shape[3] * 4)

    def activate(self, src, offset, kind, out) -> None:
        self._want(src, "activation input", (torch.float32,), 2)
        self._want(out, "activation output", (torch.float32, self.dtype), 2)
        code = _ACTIVATIONS.get(kind)
        n, w = out.shape
        if code is None or src.shape[0] != n or offset < 0 or offset + w > src.shape[1]:
            raise KernelError(f"activate: kind {kind!r}, src {tuple(src.shape)} from column {offset}, out {tuple(out.shape)}")
        self._check(self.rows.fz_activate(_p(src), c_int(src.shape[1]), c_int(offset), c_int(code), _p(out),
                                          c_int(_CODE[out.dtype]), c_int(n), c_int(w), self._stream()), "activate",
                    n * w * (4 + out.element_size()))

    def gate_multiply(self, x, gate, gate_offset, kind, out) -> None:
        self._want(x, "gated values", (self.dtype,), 2)
        self._want(out, "gated output", (self.dtype,), 2)
        self._want(gate, "gate", (torch.float32,), 2)
        code = _ACTIVATIONS.get(kind)
        n, w = x.shape
        if code is None or out.shape != x.shape or gate.shape[0] != n or gate_offset < 0 or gate_offset + w > gate.shape[1]:
            raise KernelError(f"gate_multiply: kind {kind!r}, x {tuple(x.shape)}, gate {tuple(gate.shape)} from column {gate_offset}")
        self._check(self.rows.fz_gate_multiply(_p(x), _p(gate), c_int(gate.shape[1]), c_int(gate_offset), c_int(code), _p(out),
                                               c_int(_CODE[self.dtype]), c_int(n), c_int(w), self._stream()), "gate_multiply",
                    n * w * (4 + 2 * x.element_size()))

    def blend_columns(self, dst, dst_offset, src, src_offset, width, weight) -> None:
        self._want(dst, "blend target", (torch.float32,), 2)
        self._want(src, "blend source", (torch.float32,), 2)
        self._want(weight, "blend weight", (torch.float32,), 1)
        n = dst.shape[0]
        if src.shape[0] != n or dst_offset < 0 or dst_offset + width > dst.shape[1] or src_offset < 0 or \
                src_offset + width > src.shape[1] or weight.numel() < 1:
            raise KernelError(f"blend_columns: dst {tuple(dst.shape)} from {dst_offset}, src {tuple(src.shape)} from {src_offset}, width {width}")
        self._check(self.rows.fz_blend_columns(_p(dst), c_int(dst.shape[1]), c_int(dst_offset), _p(src), c_int(src.shape[1]),
                                               c_int(src_offset), _p(weight), c_int(n), c_int(width), self._stream()),
                    "blend_columns", n * width * 12)

    def rglru_scan(self, u, gates, gate_bias, lam, y, sharpness, state, meta, out) -> None:
        self._want(u, "recurrence input", (self.dtype,), 2)
        self._want(y, "gate branch", (self.dtype,), 2)
        self._want(out, "recurrence output", (self.dtype,), 2)
        self._want(gates, "gate inputs", (torch.float32,), 3)
        self._want(gate_bias, "gate biases", (torch.float32,), 2)
        self._want(lam, "decay parameter", (torch.float32,), 1)
        self._want(state, "recurrent state", (torch.float32,), 2)
        n, w = u.shape
        parts = gates.shape[1]
        if w % parts or tuple(gates.shape) != (n, parts, 2 * (w // parts)) or tuple(gate_bias.shape) != (parts, 2 * (w // parts)) or \
                lam.shape[0] != w or y.shape != u.shape or out.shape != u.shape or state.shape[1] != w:
            raise KernelError(f"rglru_scan: u {tuple(u.shape)}, gates {tuple(gates.shape)}, bias {tuple(gate_bias.shape)}, "
                              f"lam {tuple(lam.shape)}, y {tuple(y.shape)}, state {tuple(state.shape)}")
        # long portions: the recurrence's coefficients of all rows at once, then a scan of one multiply-add per token
        cooked = int(getattr(meta, "max_portion", 0) or n) > RGLRU_COOK_ROWS
        self._meta_rows = meta.seq_row
        self._check(self.seq.fz_rglru_scan(_p(u), _p(gates), _p(gate_bias), _p(lam), _p(y), c_float(sharpness), _p(state),
                                           _p(meta.seg), c_int(getattr(meta, "max_segments", meta.n_segments)), _p(meta.seq_row),
                                           _p(out), c_int(_CODE[self.dtype]), c_int(n), c_int(w), c_int(parts), c_int(1 if cooked else 0),
                                           self._stream()), "rglru_scan", n * w * (8 + 3 * u.element_size()))
        if cooked:
            self.launches += 1

    def hashed_pair_embed(self, table, token_ids, meta, state, buckets, mul_prev, mul_cur, x) -> None:
        self._want(table, "pair table", (torch.float32, torch.bfloat16), 2)
        self._want(token_ids, "token ids", (torch.int32,), 1)
        self._want(state, "previous tokens", (torch.int32,), 2)
        self._want(x, "x", (torch.float32,), 2)
        n, d = x.shape
        if tuple(table.shape) != (buckets + 1, d) or token_ids.shape[0] != n or state.shape[1] != 1:
            raise KernelError(f"hashed_pair_embed: table {tuple(table.shape)} for {buckets} buckets, ids {tuple(token_ids.shape)}, "
                              f"x {tuple(x.shape)}, state {tuple(state.shape)}")
        self._check(self.rows.fz_hashed_pair_embed(
            _p(table), c_int(_CODE[table.dtype]), _p(token_ids), _p(meta.seq_row), _p(meta.seg), _p(state), c_int(buckets),
            c_longlong(mul_prev), c_longlong(mul_cur), c_int(2 ** 31 - 1), _p(x), c_int(n), c_int(d), _p(self.err),
            self._stream()), "hashed_pair_embed", n * d * (table.element_size() + 8))

    def depth_average(self, streams, depth, coef, x, delta) -> None:
        self._want(streams, "kept streams", (torch.float32,), 3)
        self._want(x, "x", (torch.float32,), 2)
        n, d = x.shape
        if streams.shape[0] != n or streams.shape[2] != d or not -1 <= depth < streams.shape[1] - 1 or (coef is None) != (depth == -1):
            raise KernelError(f"depth_average: streams {tuple(streams.shape)}, x {tuple(x.shape)}, depth {depth}")
        if coef is not None:
            self._want(coef, "depth weights", (torch.float32,), 1)
            if coef.shape[0] != depth + 2:
                raise KernelError(f"depth_average: {coef.shape[0]} weights at depth {depth}")
        if delta is not None:
            self._want(delta, "delta", (torch.float32,), 2)
            if delta.shape != x.shape:
                raise KernelError(f"depth_average: delta {tuple(delta.shape)} vs x {tuple(x.shape)}")
        self._check(self.rows.fz_depth_average(_p(streams), c_int(streams.shape[1]), c_int(depth), _p(coef), _p(x), _p(delta),
                                               c_int(n), c_int(d), self._stream()), "depth_average",
                    n * d * 4 * (depth + 4 + (delta is not None)))

    def depth_average_rmsnorm(self, streams, depth, coef, x, delta, weight, eps, h, rows=None) -> bool:
        if not self.fuse_depth_norm or depth < 0 or weight.dtype != torch.float32:
            return False
        self._want(streams, "kept streams", (torch.float32,), 3)
        self._want(x, "x", (torch.float32,), 2)
        self._want(coef, "depth weights", (torch.float32,), 1)
        self._want(weight, "norm weight", (torch.float32,), 1)
        self._want(h, "h", (torch.float32, torch.bfloat16), 2)
        n, d = x.shape
        n_out = n
        if rows is not None:
            self._want(rows, "rows", (torch.int32,), 1)
            n_out = rows.shape[0]
        if streams.shape[0] != n or streams.shape[2] != d or depth >= streams.shape[1] - 1 or coef.shape[0] != depth + 2 or \
                tuple(h.shape) != (n_out, d) or weight.shape[0] != d or (delta is not None and delta.shape != x.shape):
            raise KernelError(f"depth_average_rmsnorm: streams {tuple(streams.shape)}, x {tuple(x.shape)}, h {tuple(h.shape)}, depth {depth}")
        if delta is not None:
            self._want(delta, "delta", (torch.float32,), 2)
        self._check(self.rows.fz_depth_average_norm(
            _p(streams), c_int(streams.shape[1]), c_int(depth), _p(coef), _p(x), _p(delta), c_int(n), c_int(d), _p(weight),
            c_float(eps), _p(h), c_int(_CODE[h.dtype]), _p(rows), c_int(n_out), _p(self.err), self._stream()),
            "depth_average + rmsnorm", n_out * d * (4 * (depth + 3 + (delta is not None)) + h.element_size()))
        return True

    def weighted_sum(self, terms, weights, out) -> None:
        if not 1 <= len(terms) <= 4 or len(weights) != len(terms):
            raise KernelError(f"weighted_sum: {len(terms)} terms and {len(weights)} weights (1 to 4 of each)")
        self._want(out, "sum", (torch.float32,), 2)
        for t in terms:
            self._want(t, "term", (torch.float32,), 2)
            if t.shape != out.shape:
                raise KernelError(f"weighted_sum: term {tuple(t.shape)}, out {tuple(out.shape)}")
        ts = list(terms) + [None] * (4 - len(terms))
        ws = [float(w) for w in weights] + [0.0] * (4 - len(weights))
        self._check(self.seq.fz_weighted_sum(*(_p(t) for t in ts), *(c_float(w) for w in ws), c_int(len(terms)), _p(out),
                                             c_longlong(out.numel()), self._stream()), "weighted_sum",
                    out.numel() * 4 * (len(terms) + 1))

    def route_by_scores(self, logits, num_experts, top, groups, keep_groups, renormalize, meta, weights, align: int = 1):
        self._want(logits, "router logits", (torch.float32,), 2)
        self._want(weights, "router weights", (torch.float32,), 2)
        n = logits.shape[0]
        if logits.shape[1] < num_experts or tuple(weights.shape) != (n, top):
            raise KernelError(f"route_by_scores: logits {tuple(logits.shape)}, weights {tuple(weights.shape)}, {num_experts} experts")
        choice = self._scratch("router choices", max(n, 1) * top, torch.int32)[:n * top].view(n, top)
        self._check(self.seq.fz_router_topk(_p(logits), c_int(logits.shape[1]), c_int(n), c_int(num_experts), c_int(top),
                                            c_int(groups), c_int(keep_groups), c_int(1 if renormalize else 0), _p(meta.seq_row),
                                            _p(choice), _p(weights), self._stream()), "router_topk")
        self._meta_rows = meta.seq_row
        return self._sort_pairs(None, n, meta, choice, num_experts, align)

    def moe_combine(self, terms, weights, shared, gate_logits, gate_column, out, add=None, scale: float = 1.0) -> None:
        self._want(terms, "expert terms", (torch.float32,), 2)
        self._want(weights, "router weights", (torch.float32,), 2)
        self._want(out, "feed-forward output", (torch.float32,), 2)
        n, top = weights.shape
        d = out.shape[1]
        if tuple(terms.shape) != (n * top, d) or out.shape[0] != n:
            raise KernelError(f"moe_combine: terms {tuple(terms.shape)}, weights {tuple(weights.shape)}, out {tuple(out.shape)}")
        ldg = 0
        if shared is not None:
            self._want(shared, "shared expert output", (torch.float32,), 2)
            if shared.shape != out.shape:
                raise KernelError(f"moe_combine: shared {tuple(shared.shape)}, out {tuple(out.shape)}")
            if gate_logits is not None:
                self._want(gate_logits, "shared gate logits", (torch.float32,), 2)
                ldg = gate_logits.shape[1]
                if gate_logits.shape[0] != n or not 0 <= gate_column < ldg:
                    raise KernelError(f"moe_combine: gate logits {tuple(gate_logits.shape)} column {gate_column}")
        else:
            gate_logits = None
        if add is not None:
            self._want(add, "other term", (torch.float32,), 2)
            if add.shape != out.shape:
                raise KernelError(f"moe_combine: other term {tuple(add.shape)}, out {tuple(out.shape)}")
        self._check(self.seq.fz_moe_combine(_p(terms), _p(weights), c_int(top), _p(shared), _p(gate_logits), c_int(ldg),
                                            c_int(gate_column), _p(self._step_rows(n)), _p(out), c_int(n), c_int(d), _p(add), c_float(scale),
                                            self._stream()),
                    "moe_combine", n * d * 4 * (top + 1 + (shared is not None) + (add is not None)))
