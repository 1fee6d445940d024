"""Synthetic weight sets and the client call stream that loads them.

The reference measures its swap path on torchvision / Hugging Face checkpoints
served from PyTorch client containers (tests/endpoint.py:16-40).  Those files
are not needed for a byte-movement path: what matters is the list of tensor
sizes, the order a client uploads and first touches them, and how the client's
caching allocator groups them into device blocks.  This module rebuilds those
three things from the architecture dimensions alone.

* ``weight_set(name)``        -- tensors of a model in module order
* ``tensor_bytes(ws, i, seed)``-- seeded N(0, 0.02) values of tensor ``i``
* ``pack_blocks(ws)``         -- client-allocator emulation: which device block
                                 (size, offset) every tensor is uploaded into
* ``cold_start_stream(ws)``   -- the malloc / memcpy / first-access call stream
                                 an executor receives for one function
                                 (include/server/cuda_server.hpp:951-978,1027-1037)
"""
from __future__ import annotations

import dataclasses
from concurrent.futures import ThreadPoolExecutor
from typing import Iterator, List, Sequence, Tuple

import numpy as np

MiB = 1 << 20

# Block sizes a PyTorch client sends to cudaMalloc; the reference's pool has
# dedicated size classes for the first two (include/server/block_manager.hpp:28-30).
SMALL_BLOCK = 2 * MiB      # tensors <= 1 MiB are packed into 2 MiB blocks
LARGE_BLOCK = 20 * MiB     # 1 MiB < tensor < 10 MiB are packed into 20 MiB blocks
SMALL_LIMIT = 1 * MiB
LARGE_LIMIT = 10 * MiB
PACK_ALIGN = 512
ROUND_LARGE = 2 * MiB      # tensors >= 10 MiB get their own block, rounded to 2 MiB


@dataclasses.dataclass(frozen=True)
class Tensor:
    name: str
    shape: Tuple[int, ...]
    dtype: str  # "float32" | "float16"

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    @property
    def nbytes(self) -> int:
        return self.numel * (4 if self.dtype == "float32" else 2)


@dataclasses.dataclass(frozen=True)
class WeightSet:
    name: str
    seed: int
    tensors: Tuple[Tensor, ...]

    @property
    def nbytes(self) -> int:
        return sum(t.nbytes for t in self.tensors)

    @property
    def numel(self) -> int:
        return sum(t.numel for t in self.tensors)


def _resnet50(dtype: str) -> List[Tensor]:
    out: List[Tensor] = []

    def conv(name, cout, cin, k):
        out.append(Tensor(name + ".weight", (cout, cin, k, k), dtype))

    def bn(name, c):
        out.append(Tensor(name + ".weight", (c,), dtype))
        out.append(Tensor(name + ".bias", (c,), dtype))

    conv("conv1", 64, 3, 7)
    bn("bn1", 64)
    inplanes = 64
    for li, (planes, blocks) in enumerate(zip((64, 128, 256, 512), (3, 4, 6, 3)), start=1):
        for b in range(blocks):
            p = f"layer{li}.{b}"
            conv(p + ".conv1", planes, inplanes, 1)
            bn(p + ".bn1", planes)
            conv(p + ".conv2", planes, planes, 3)
            bn(p + ".bn2", planes)
            conv(p + ".conv3", planes * 4, planes, 1)
            bn(p + ".bn3", planes * 4)
            if b == 0:
                conv(p + ".downsample.0", planes * 4, inplanes, 1)
                bn(p + ".downsample.1", planes * 4)
            inplanes = planes * 4
    out.append(Tensor("fc.weight", (1000, 2048), dtype))
    out.append(Tensor("fc.bias", (1000,), dtype))
    return out


def _vgg19(dtype: str) -> List[Tensor]:
    cfg = [64, 64, "M", 128, 128, "M", 256, 256, 256, 256, "M", 512, 512, 512, 512, "M", 512, 512, 512, 512, "M"]
    out: List[Tensor] = []
    cin, idx = 3, 0
    for v in cfg:
        if v == "M":
            idx += 1
            continue
        out.append(Tensor(f"features.{idx}.weight", (v, cin, 3, 3), dtype))
        out.append(Tensor(f"features.{idx}.bias", (v,), dtype))
        cin = v
        idx += 2
    for i, (o, n) in zip((0, 3, 6), ((4096, 512 * 7 * 7), (4096, 4096), (1000, 4096))):
        out.append(Tensor(f"classifier.{i}.weight", (o, n), dtype))
        out.append(Tensor(f"classifier.{i}.bias", (o,), dtype))
    return out


def _bert(dtype: str, layers: int, hidden: int, ffn: int, vocab: int = 30522, max_pos: int = 512) -> List[Tensor]:
    out: List[Tensor] = []

    def lin(name, o, i):
        out.append(Tensor(name + ".weight", (o, i), dtype))
        out.append(Tensor(name + ".bias", (o,), dtype))

    def ln(name):
        out.append(Tensor(name + ".weight", (hidden,), dtype))
        out.append(Tensor(name + ".bias", (hidden,), dtype))

    out.append(Tensor("embeddings.word_embeddings.weight", (vocab, hidden), dtype))
    out.append(Tensor("embeddings.position_embeddings.weight", (max_pos, hidden), dtype))
    out.append(Tensor("embeddings.token_type_embeddings.weight", (2, hidden), dtype))
    ln("embeddings.LayerNorm")
    for l in range(layers):
        p = f"encoder.layer.{l}"
        lin(p + ".attention.self.query", hidden, hidden)
        lin(p + ".attention.self.key", hidden, hidden)
        lin(p + ".attention.self.value", hidden, hidden)
        lin(p + ".attention.output.dense", hidden, hidden)
        ln(p + ".attention.output.LayerNorm")
        lin(p + ".intermediate.dense", ffn, hidden)
        lin(p + ".output.dense", hidden, ffn)
        ln(p + ".output.LayerNorm")
    lin("pooler.dense", hidden, hidden)
    return out


def _llama(dtype: str, layers: int = 32, hidden: int = 4096, ffn: int = 11008, vocab: int = 32000) -> List[Tensor]:
    out: List[Tensor] = [Tensor("model.embed_tokens.weight", (vocab, hidden), dtype)]
    for l in range(layers):
        p = f"model.layers.{l}"
        for proj in ("q_proj", "k_proj", "v_proj", "o_proj"):
            out.append(Tensor(f"{p}.self_attn.{proj}.weight", (hidden, hidden), dtype))
        out.append(Tensor(f"{p}.mlp.gate_proj.weight", (ffn, hidden), dtype))
        out.append(Tensor(f"{p}.mlp.up_proj.weight", (ffn, hidden), dtype))
        out.append(Tensor(f"{p}.mlp.down_proj.weight", (hidden, ffn), dtype))
        out.append(Tensor(f"{p}.input_layernorm.weight", (hidden,), dtype))
        out.append(Tensor(f"{p}.post_attention_layernorm.weight", (hidden,), dtype))
    out.append(Tensor("model.norm.weight", (hidden,), dtype))
    out.append(Tensor("lm_head.weight", (vocab, hidden), dtype))
    return out


_BUILDERS = {
    # name: (builder, dtype, seed)  -- the five shapes named by the benchmark configuration
    "resnet50": (lambda d: _resnet50(d), "float32", 0),
    "bert_base": (lambda d: _bert(d, 12, 768, 3072), "float32", 1),
    "bert_large": (lambda d: _bert(d, 24, 1024, 4096), "float16", 2),
    "llama2_7b": (lambda d: _llama(d), "float16", 3),
    "vgg19": (lambda d: _vgg19(d), "float32", 4),
    # reduced shapes for fast tests (same structure, fewer/lighter layers)
    "bert_tiny": (lambda d: _bert(d, 2, 128, 512, vocab=4096, max_pos=128), "float32", 11),
    "llama_tiny": (lambda d: _llama(d, layers=2, hidden=1024, ffn=2752, vocab=8000), "float16", 12),
    "llama_mid": (lambda d: _llama(d, layers=4, hidden=4096, ffn=11008, vocab=32000), "float16", 13),
}


def weight_set(name: str, seed: int | None = None) -> WeightSet:
    builder, dtype, default_seed = _BUILDERS[name]
    return WeightSet(name, default_seed if seed is None else seed, tuple(builder(dtype)))


def tensor_values(ws: WeightSet, index: int) -> np.ndarray:
    """Tensor ``index`` of ``ws``: N(0, 0.02) drawn in float32 from the stream
    ``default_rng([seed, index])`` and cast to the set's dtype.  One stream per
    tensor keeps every tensor reproducible on its own, so large sets can be
    generated in parallel and checked piecewise."""
    t = ws.tensors[index]
    rng = np.random.default_rng([ws.seed, index])
    v = rng.standard_normal(t.numel, dtype=np.float32)
    v *= np.float32(0.02)
    if t.dtype == "float16":
        return v.astype(np.float16)
    return v


def tensor_bytes(ws: WeightSet, index: int) -> np.ndarray:
    return tensor_values(ws, index).view(np.uint8)


def generate_into(ws: WeightSet, sink, threads: int = 8) -> None:
    """Call ``sink(index, uint8_array)`` for every tensor, generating with a thread pool
    (numpy's generators release the GIL)."""
    def job(i):
        sink(i, tensor_bytes(ws, i))
    with ThreadPoolExecutor(max_workers=max(1, threads)) as ex:
        list(ex.map(job, range(len(ws.tensors))))


# ------------------------------------------------------------------ packing

@dataclasses.dataclass
class PackedBlock:
    size: int
    is_model: bool
    used: int = 0
    params: List[Tuple[int, int]] = dataclasses.field(default_factory=list)  # (tensor index, offset)


def pack_blocks(ws: WeightSet) -> Tuple[List[PackedBlock], List[Tuple[int, int]]]:
    """Group tensors into device blocks the way a PyTorch client's caching
    allocator would ask the server for them: small tensors share 2 MiB blocks,
    medium ones share 20 MiB blocks (both at 512-byte alignment, first fit in
    arrival order), anything of 10 MiB or more gets its own block rounded up to
    2 MiB.  Returns the blocks in creation order and, per tensor, (block, offset)."""
    blocks: List[PackedBlock] = []
    where: List[Tuple[int, int]] = []
    small: List[int] = []
    large: List[int] = []
    for i, t in enumerate(ws.tensors):
        n = t.nbytes
        if n >= LARGE_LIMIT:
            size = (n + ROUND_LARGE - 1) // ROUND_LARGE * ROUND_LARGE
            blocks.append(PackedBlock(size, True, n, [(i, 0)]))
            where.append((len(blocks) - 1, 0))
            continue
        pool, bsize = (small, SMALL_BLOCK) if n <= SMALL_LIMIT else (large, LARGE_BLOCK)
        need = (n + PACK_ALIGN - 1) // PACK_ALIGN * PACK_ALIGN
        placed = False
        for b in pool:
            if blocks[b].used + need <= bsize:
                off = blocks[b].used
                blocks[b].params.append((i, off))
                blocks[b].used += need
                where.append((b, off))
                placed = True
                break
        if not placed:
            blocks.append(PackedBlock(bsize, True, need, [(i, 0)]))
            pool.append(len(blocks) - 1)
            where.append((len(blocks) - 1, 0))
    return blocks, where


@dataclasses.dataclass(frozen=True)
class Call:
    """One call of the cold-start stream.  ``op`` is one of
    malloc / memcpy / sync_done / access; ``block`` indexes the block list of
    ``pack_blocks`` (or -1 - k for the k-th non-model block), ``tensor`` the tensor."""
    op: str
    block: int = 0
    tensor: int = -1
    offset: int = 0
    size: int = 0
    is_model: bool = True


def cold_start_stream(ws: WeightSet, workspace_blocks: Sequence[int] = (SMALL_BLOCK,)) -> Iterator[Call]:
    """The call stream an executor sees while a client loads ``ws`` and runs once:
    ``model.cuda()`` interleaves block mallocs with per-tensor uploads; the
    synchronize that follows marks the end of the model; later mallocs are
    activation / workspace blocks; the first inference touches every tensor in
    module order."""
    blocks, where = pack_blocks(ws)
    seen = set()
    for i, t in enumerate(ws.tensors):
        b, off = where[i]
        if b not in seen:
            seen.add(b)
            yield Call("malloc", block=b, size=blocks[b].size, is_model=True)
        yield Call("memcpy", block=b, tensor=i, offset=off, size=t.nbytes)
    yield Call("sync_done")
    for k, size in enumerate(workspace_blocks):
        yield Call("malloc", block=-1 - k, size=size, is_model=False)
    for i in range(len(ws.tensors)):
        b, off = where[i]
        yield Call("access", block=b, tensor=i, offset=off)


# ------------------------------------------------------------- request mix

def mixed_stream(seed: int = 4, n_models: int = 64, rate: float = 200.0, duration_s: float = 120.0,
                 zipf_s: float = 1.1, archs: Sequence[str] = ("resnet50", "bert_base", "bert_large", "vgg19")):
    """The serverless request mix: ``n_models`` functions whose architectures are
    drawn uniformly from ``archs``; request popularity Zipf(s) over a random
    permutation of the functions; Poisson arrivals at ``rate`` requests/s for
    ``duration_s`` seconds (the generator shape of scripts/sender_fix_rate.py:46-56).
    Returns (arch_of_model, arrival_times, model_of_request)."""
    rng = np.random.default_rng(seed)
    arch_idx = rng.integers(0, len(archs), size=n_models)
    perm = rng.permutation(n_models)
    ranks = np.arange(1, n_models + 1, dtype=np.float64)
    p = ranks ** (-zipf_s)
    p /= p.sum()
    n_expected = int(rate * duration_s * 1.2) + 16
    gaps = rng.exponential(1.0 / rate, size=n_expected)
    times = np.cumsum(gaps)
    times = times[times < duration_s]
    picks = rng.choice(n_models, size=times.shape[0], p=p)
    return [archs[a] for a in arch_idx], times, perm[picks]


# ------------------------------------------------------------- cold start

@dataclasses.dataclass
class LoadedModel:
    func: str
    ws: WeightSet
    block_vaddr: List[int]          # per packed block
    workspace_vaddr: List[int]      # per non-model block
    tensor_vaddr: List[int]         # per tensor: the client-visible ("virtual") device pointer


def cold_start(mgr, func: str, ws: WeightSet, tensor_data=None,
               workspace_blocks: Sequence[int] = (SMALL_BLOCK,)) -> LoadedModel:
    """Replay the cold-start call stream of ``ws`` into a memory manager.

    ``mgr`` is anything with the executor-facing methods of the reference's
    MemoryManager under their short names (track_begin, malloc, memcpy_h2d_model,
    sync_done, mark_access, track_end) -- the shipped engine and both checkers
    expose them.  ``tensor_data(i)`` returns tensor ``i`` as a uint8 array
    (default: the seeded values)."""
    if tensor_data is None:
        tensor_data = lambda i: tensor_bytes(ws, i)
    blocks, _ = pack_blocks(ws)
    bv = [0] * len(blocks)
    wv: List[int] = []
    tv = [0] * len(ws.tensors)
    mgr.track_begin(func)
    for c in cold_start_stream(ws, workspace_blocks):
        if c.op == "malloc":
            p = mgr.malloc(func, c.size, c.is_model)
            if c.is_model:
                bv[c.block] = p
            else:
                wv.append(p)
        elif c.op == "memcpy":
            tv[c.tensor] = bv[c.block] + c.offset
            rc = mgr.memcpy_h2d_model(func, tv[c.tensor], tensor_data(c.tensor))
            if rc != 0:
                raise RuntimeError(f"upload of tensor {c.tensor} of {func} was not recorded (rc={rc})")
        elif c.op == "sync_done":
            mgr.sync_done(func)
        elif c.op == "access":
            mgr.mark_access(tv[c.tensor])
    mgr.track_end(func)
    return LoadedModel(func, ws, bv, wv, tv)


# ------------------------------------------------------------- sizing helpers

def pool_budget_for(ws: WeightSet, workspace_blocks: Sequence[int] = (SMALL_BLOCK,), slack_chunks: int = 6) -> int:
    """A memory budget (the engine adds the reference's hidden 5 GiB to it) whose pool of
    128 MiB chunks holds ``ws`` once: 2 MiB / 20 MiB blocks as they are, other blocks up to a
    chunk rounded to a power of two of at least 16 MiB, larger ones outside the pool."""
    chunk = 128 * MiB
    regular = irregular = 0
    for size in [b.size for b in pack_blocks(ws)[0]] + list(workspace_blocks):
        if size in (SMALL_BLOCK, LARGE_BLOCK):
            regular += size if size == SMALL_BLOCK else chunk // 6 + 1   # six 20 MiB windows per chunk
        elif size <= chunk:
            r = 16 * MiB
            while r < size:
                r *= 2
            irregular += r
    chunks = -(-regular // chunk) + -(-irregular // chunk) + slack_chunks
    return max(0, chunks * chunk - (5 << 30))


def host_store_bytes(ws: WeightSet) -> int:
    """Bytes of page-locked host store one copy of ``ws`` needs (block mirrors, 4 KiB aligned)."""
    total = sum((b.size + 4095) // 4096 * 4096 for b in pack_blocks(ws)[0])
    return ((total >> 30) + 1) << 30


def plan_tables(ws: WeightSet, func: str, *, budget: int, target_server: int = 0, holder_server: int = 0,
                gpu_count: int = 1, swaps: int = 1, block_manager: str = "Buddy"):
    """Block and pointer tables (canonical addresses) that the target engine must show after each of
    ``swaps`` swap-ins of ``ws`` with an eviction between them, worked out on plan-only engines: the
    same placement and rebind decisions, no byte moved, no GPU needed.  ``holder_server`` is the
    engine that cold-starts the model (the target itself evicts it first when they are the same).
    Uses the process-wide model repository: call it while no other engine holds ``func``.
    Returns a list of (blocks, params) pairs, one per swap-in."""
    from .memory_manager import MemoryManager, SizeOnly
    engines = {}
    for sid in sorted({target_server, holder_server}):
        engines[sid] = MemoryManager(budget, device=-1, server_id=sid, gpu_count=gpu_count, block_manager=block_manager)
    out = []
    try:
        cold_start(engines[holder_server], func, ws, tensor_data=lambda i: SizeOnly(ws.tensors[i].nbytes))
        target = engines[target_server]
        if holder_server == target_server:
            target.evict(func)
        for _ in range(swaps):
            target.swap_in(func, -1)
            out.append((target.dump_blocks(func, canonical=True), target.dump_params(func, canonical=True)))
            target.evict(func)
    finally:
        for e in engines.values():
            e.close()
    return out
