"""Multi-GPU sharding of the render path on one node (one process per GPU, ``torch.distributed``).

Two shardings, neither of which exists in the reference (its ``gsplat/distributed.py`` is a bag of
helper collectives with no caller in ``rendering.py``; the pattern followed here is its
size exchange + row all-to-all, ``distributed.py:170-257``):

1. **Sensors split, Gaussians replicated** - every rank holds all N Gaussians and renders the
   sensors :func:`sensor_owners` assigns to it with the single-GPU path. Sensors are independent,
   so the forward data path has no collective at all (:func:`all_reduce_gradients` sums the
   parameter gradients when training).

2. **Gaussians split, projected records routed to the sensor's owner**
   (:func:`rasterization_gaussian_sharded`, :func:`lidar_rasterization_gaussian_sharded`) - rank r
   holds a contiguous slice of the Gaussians (:func:`gaussian_slice`) and projects it against ALL
   sensors, taken in *send order* (grouped by owner rank, :func:`sensor_send_order`). Per step:

   * ``visible_rows`` (device): which (sensor, Gaussian) pairs travel, in (sensor, Gaussian) order,
     and how many per sensor;
   * one ``all_gather`` of the per-sensor counts and ONE host synchronisation: NCCL needs the split
     sizes on the host (:func:`plan_exchange` turns the count matrix into split sizes and the
     segment table of the receive buffer);
   * ``pack_rows`` (device): one fixed-width row of 32-bit words per travelling pair, gathered
     straight from the [C, N_local] projection outputs: 2 ids + radii 2 + means2d 2 + depth 1 +
     conic 3 + opacity 1 + pixel velocity 2 + colour D for cameras (68 B at D = 4 with the depth
     channel); lidars carry velocity 3, depth compensation 2 and D features (128 B at D = 16);
   * ONE ``all_to_all_single`` of the rows over NVLink (differentiable: the backward pass is the
     mirrored all-to-all of the row gradients);
   * ``unpack_rows`` (device): rows land in (sensor, global Gaussian id) order - exactly the packed
     layout a single GPU produces, so tile lists and tie-breaks are those of a single-GPU run -
     through a row map built from the segment table (no sort).

   The owner then runs tile intersection and compositing in the packed layout.

NCCL moves the rows into local HBM; kernels only ever read local memory (no peer loads, no
multicast). The host-side planning and the differentiable all-to-all also run with the gloo
backend on CPU tensors, which is how they are tested without GPUs; packing, placing and rendering
need the CUDA library.
"""

from __future__ import annotations

import ctypes
import math
from typing import Dict, List, NamedTuple, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
import torch.distributed.nn.functional as distF
from torch import Tensor


class PeerLostError(RuntimeError):
    """A collective of the exchange failed or timed out: a peer rank has gone away."""


def sensor_owners(n_sensors: int, world_size: int, costs: Optional[Sequence[float]] = None) -> List[int]:
    """Owner rank of every sensor. Without ``costs``: round-robin. With per-sensor cost estimates
    (e.g. pixels or points per sensor): longest-processing-time-first onto the least loaded rank,
    ties to the lower rank, so a 2-Mpixel camera and a 0.23-Mpoint lidar do not weigh the same."""
    if costs is None:
        return [c % world_size for c in range(n_sensors)]
    assert len(costs) == n_sensors
    load = [0.0] * world_size
    owner = [0] * n_sensors
    for c in sorted(range(n_sensors), key=lambda i: (-costs[i], i)):
        r = min(range(world_size), key=lambda k: (load[k], k))
        owner[c] = r
        load[r] += float(costs[c])
    return owner


def local_sensors(owners: Sequence[int], rank: int) -> List[int]:
    return [c for c, r in enumerate(owners) if r == rank]


def gaussian_slice(n_gaussians: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Contiguous [start, end) slice of the Gaussians held by ``rank`` (sizes differ by at most 1)."""
    base, rem = divmod(n_gaussians, world_size)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def sensor_send_order(owners: Sequence[int]) -> List[int]:
    """Sensors grouped by owner rank (ascending sensor id inside a group): projected in this order,
    the travelling rows of a rank are already laid out as one contiguous block per destination."""
    return sorted(range(len(owners)), key=lambda c: (owners[c], c))


def _world(group) -> Tuple[int, int]:
    if not dist.is_available() or not dist.is_initialized():
        return 1, 0
    return dist.get_world_size(group), dist.get_rank(group)


class ExchangePlan(NamedTuple):
    """Host-side description of one exchange, from the [world, C] matrix of travelling rows per
    (source rank, sensor in send order)."""
    send_splits: List[int]   # rows this rank sends to every rank
    recv_splits: List[int]   # rows this rank receives from every rank
    mine: List[int]          # global ids of the sensors this rank owns, ascending
    src_start: List[int]     # segment starts in the receive buffer, (source, sensor) order; total last
    dst_start: List[int]     # the same segments' starts in the final (sensor, source) order
    sensor_start: List[int]  # first final row of every owned sensor; total last


def plan_exchange(counts: Sequence[Sequence[int]], order: Sequence[int], owners: Sequence[int],
                  rank: int) -> ExchangePlan:
    """Split sizes and segment table of rank ``rank`` for the count matrix ``counts[source][p]``
    (``p`` indexes sensors in send order ``order``)."""
    world = len(counts)
    dest = [owners[c] for c in order]
    send_splits = [sum(int(counts[rank][p]) for p in range(len(order)) if dest[p] == d) for d in range(world)]
    my_pos = [p for p in range(len(order)) if dest[p] == rank]
    recv_splits = [sum(int(counts[s][p]) for p in my_pos) for s in range(world)]
    # receive buffer: for every source, its rows for my sensors in ascending sensor order
    src_start, run = [], 0
    for s in range(world):
        for p in my_pos:
            src_start.append(run)
            run += int(counts[s][p])
    src_start.append(run)
    # final order: for every sensor of mine, the sources in rank order (= ascending global Gaussian id)
    final, run, sensor_start = {}, 0, []
    for p in my_pos:
        sensor_start.append(run)
        for s in range(world):
            final[(s, p)] = run
            run += int(counts[s][p])
    sensor_start.append(run)
    dst_start = [final[(s, p)] for s in range(world) for p in my_pos]
    return ExchangePlan(send_splits, recv_splits, [order[p] for p in my_pos], src_start, dst_start, sensor_start)


def exchange_rows(rows: Tensor, send_splits: Sequence[int], recv_splits: Sequence[int], group=None) -> Tensor:
    """One differentiable all-to-all of ``rows`` [sum(send_splits), W]; returns [sum(recv_splits), W]
    with the blocks of the source ranks in rank order. A failed or timed-out collective (a peer that
    left) surfaces as :class:`PeerLostError` instead of a backend-specific exception."""
    world, _ = _world(group)
    if world == 1:
        return rows
    out = torch.empty((int(sum(recv_splits)), rows.shape[1]), dtype=rows.dtype, device=rows.device)
    try:
        return distF.all_to_all_single(out, rows.contiguous(), list(recv_splits), list(send_splits), group=group)
    except (RuntimeError, ValueError) as e:   # DistBackendError derives from RuntimeError
        raise PeerLostError(f"row exchange failed: {e}") from e


def gather_counts(indptr: Tensor, group=None) -> List[List[int]]:
    """The [world, C] matrix of travelling rows per (rank, sensor) from every rank's device
    ``indptr`` [C + 1]: one all_gather and the step's one host synchronisation."""
    world, _ = _world(group)
    counts = (indptr[1:] - indptr[:-1]).to(torch.int64)
    if world == 1:
        return [counts.tolist()]
    gathered = torch.empty((world, counts.numel()), dtype=torch.int64, device=indptr.device)
    try:
        dist.all_gather_into_tensor(gathered, counts.contiguous(), group=group)
        return gathered.tolist()
    except (RuntimeError, ValueError) as e:
        raise PeerLostError(f"count exchange failed: {e}") from e


# ---------------------------------------------------------------------------------------------
# Device ops of the exchange (CUDA library, no CPU fallback)
# ---------------------------------------------------------------------------------------------
def _tables(ptrs: Sequence[Optional[int]], widths: Sequence[int]):
    n = len(widths)
    p = (ctypes.c_void_p * max(n, 1))(*[None if x is None else int(x) for x in ptrs])
    w = (ctypes.c_int32 * max(n, 1))(*[int(x) for x in widths])
    return p, w


def visible_rows(radii: Tensor) -> Tuple[Tensor, Tensor]:
    """Travelling pairs of a [C, N, 2] radii tensor (float degrees or int32 pixels): returns
    (row_index int32 [C * N] whose first ``indptr[C]`` entries are the pair indices c * N + n in
    (sensor, Gaussian) order, indptr int32 [C + 1] on the device). Nothing is read back."""
    from . import _lib
    C, N = radii.shape[:2]
    assert radii.shape == (C, N, 2) and radii.dtype in (torch.float32, torch.int32), (radii.shape, radii.dtype)
    radii = radii.contiguous()
    dev = radii.device
    indptr = torch.zeros(C + 1, dtype=torch.int32, device=dev)
    row_index = torch.empty(max(C * N, 1), dtype=torch.int32, device=dev)
    if C == 0 or N == 0:
        return row_index, indptr
    lib = _lib.load()
    ws = _lib.workspace("visible_rows", lib.splatad_visible_rows_workspace_bytes(C, N), dev)
    stream = _lib.stream_ptr(dev)
    _lib.call("splatad_visible_rows_count", C, N, _lib.ptr(radii), _lib.ptr(ws), ws.numel(), _lib.ptr(indptr),
              None, stream)
    _lib.call("splatad_visible_rows_fill", C, N, _lib.ptr(radii), _lib.ptr(ws), row_index.numel(),
              _lib.ptr(row_index), stream)
    return row_index, indptr


def _words(t: Tensor) -> Tensor:
    assert t.dtype in (torch.float32, torch.int32), t.dtype
    return t.contiguous()


class _PackRows(torch.autograd.Function):
    """rows[i] = (global sensor id, global Gaussian id, fields of pair row_index[i] ...)."""

    @staticmethod
    def forward(ctx, row_index, n_rows, sensor_table, n_per_sensor, gaussian_start, *fields):
        from . import _lib
        fields = [_words(f) for f in fields]
        widths = [int(f.shape[1]) for f in fields]   # fields are [pairs, width] views
        dev = fields[0].device
        out = torch.empty((n_rows, 2 + sum(widths)), dtype=torch.float32, device=dev)
        ptrs, w = _tables([_lib.ptr(f) for f in fields], widths)
        if n_rows:
            _lib.call("splatad_rows_gather", n_rows, _lib.ptr(row_index), len(fields), ctypes.addressof(ptrs),
                      ctypes.addressof(w), _lib.ptr(sensor_table), n_per_sensor, gaussian_start, _lib.ptr(out),
                      _lib.stream_ptr(dev))
        ctx.save_for_backward(row_index)
        ctx.meta = (n_rows, widths, [tuple(f.shape) for f in fields], [f.dtype for f in fields])
        return out

    @staticmethod
    def backward(ctx, v_rows):
        from . import _lib
        (row_index,) = ctx.saved_tensors
        n_rows, widths, shapes, dtypes = ctx.meta
        dev = v_rows.device
        grads = [torch.zeros(shape, dtype=torch.float32, device=dev)
                 if (ctx.needs_input_grad[5 + k] and dtypes[k] == torch.float32) else None
                 for k, shape in enumerate(shapes)]
        if n_rows and any(g is not None for g in grads):
            ptrs, w = _tables([None if g is None else _lib.ptr(g) for g in grads], widths)
            _lib.call("splatad_rows_scatter", n_rows, _lib.ptr(row_index), len(widths), ctypes.addressof(ptrs),
                      ctypes.addressof(w), 2, None, None, _lib.ptr(v_rows.contiguous()), _lib.stream_ptr(dev))
        return (None, None, None, None, None, *grads)


class _UnpackRows(torch.autograd.Function):
    """Places received rows: field_k[row_map[i]] = columns of field k of rows[i]."""

    @staticmethod
    def forward(ctx, rows, row_map, widths, int_fields):
        from . import _lib
        rows = rows.contiguous()
        n_rows, dev = rows.shape[0], rows.device
        assert rows.shape[1] == 2 + sum(widths), (rows.shape, widths)
        sensor_ids = torch.empty(n_rows, dtype=torch.int64, device=dev)
        gaussian_ids = torch.empty(n_rows, dtype=torch.int64, device=dev)
        outs = [torch.empty((n_rows, w), dtype=torch.int32 if is_int else torch.float32, device=dev)
                for w, is_int in zip(widths, int_fields)]
        if n_rows:
            ptrs, w = _tables([_lib.ptr(o) for o in outs], widths)
            _lib.call("splatad_rows_scatter", n_rows, _lib.ptr(row_map), len(widths), ctypes.addressof(ptrs),
                      ctypes.addressof(w), 2, _lib.ptr(sensor_ids), _lib.ptr(gaussian_ids), _lib.ptr(rows),
                      _lib.stream_ptr(dev))
        ctx.save_for_backward(row_map)
        ctx.meta = (n_rows, tuple(widths), tuple(int_fields))
        ctx.mark_non_differentiable(sensor_ids, gaussian_ids, *[o for o, i in zip(outs, int_fields) if i])
        return (sensor_ids, gaussian_ids, *outs)

    @staticmethod
    def backward(ctx, v_sensor_ids, v_gaussian_ids, *v_fields):
        from . import _lib
        (row_map,) = ctx.saved_tensors
        n_rows, widths, int_fields = ctx.meta
        dev = row_map.device
        v_rows = torch.empty((n_rows, 2 + sum(widths)), dtype=torch.float32, device=dev)
        if n_rows:
            srcs = [None if (v is None or is_int) else v.contiguous() for v, is_int in zip(v_fields, int_fields)]
            # a leading width-2 field without a source stands for the id columns (zeros)
            ptrs, w = _tables([None] + [None if s is None else _lib.ptr(s) for s in srcs], (2,) + widths)
            _lib.call("splatad_rows_gather", n_rows, _lib.ptr(row_map), len(widths) + 1, ctypes.addressof(ptrs),
                      ctypes.addressof(w), None, 0, 0, _lib.ptr(v_rows), _lib.stream_ptr(dev))
        return v_rows, None, None, None


def segment_row_map(plan: ExchangePlan, device) -> Tuple[Tensor, Tensor]:
    """(row_map int32 [n_received]: final row of every received row; local_sensor_ids int64
    [n_received]: per final row, the index of its sensor among the sensors this rank owns), from the
    plan's segment table, which travels in the kernel's arguments."""
    from . import _lib
    device = torch.device(device)
    n_rows = plan.src_start[-1]
    row_map = torch.empty(n_rows, dtype=torch.int32, device=device)
    local_ids = torch.empty(n_rows, dtype=torch.int64, device=device)
    n_seg = len(plan.dst_start)
    if n_rows == 0 or n_seg == 0:
        return row_map, local_ids
    src = (ctypes.c_int64 * n_seg)(*plan.src_start[:n_seg])
    dst = (ctypes.c_int64 * n_seg)(*plan.dst_start)
    _lib.call("splatad_segment_row_map", n_seg, max(len(plan.mine), 1), ctypes.addressof(src), ctypes.addressof(dst),
              n_rows, _lib.ptr(row_map), _lib.ptr(local_ids), _lib.stream_ptr(device))
    return row_map, local_ids


_device_constants: Dict[tuple, Tensor] = {}


def _device_ints(values: Sequence[int], dtype, device) -> Tensor:
    """Small constant integer tables (sensor orders, owned sensor lists) on the device, uploaded once."""
    key = (tuple(int(v) for v in values), dtype, str(device))
    t = _device_constants.get(key)
    if t is None:
        t = torch.tensor(list(key[0]), dtype=dtype, device=device)
        _device_constants[key] = t
    return t


def exchange_projected(
    fields: Dict[str, Tensor],   # name -> [C, N_local, ...] float32 / int32, sensors in SEND order
    radii: Tensor,               # [C, N_local, 2]: pairs with radii[..., 0] > 0 travel (sent as field "radii")
    gaussian_start: int,         # global id of local Gaussian 0
    owners: Sequence[int],       # owner rank of every sensor (global sensor ids)
    order: Sequence[int],        # send order: position p holds global sensor order[p]
    group=None,
    stats: Optional[dict] = None,
) -> Tuple[Dict[str, Tensor], Tensor, Tensor, ExchangePlan]:
    """Routes the visible records to the ranks owning their sensors.

    Returns ``(received, sensor_ids, gaussian_ids, plan)``: for every field (and ``"radii"``, plus
    ``"local_sensor_ids"``, int64) a ``[nnz_r, ...]`` tensor of the rows this rank received, ordered by (global sensor id, global
    Gaussian id) - the packed layout of a single-GPU run restricted to this rank's sensors -, the
    int64 global sensor / Gaussian ids of the rows, and the exchange plan. Differentiable with
    respect to every float field. ``stats`` (optional dict) receives the bytes put on the wire.
    """
    world, rank = _world(group)
    C, n_local = radii.shape[:2]
    dev = radii.device
    names = ["radii"] + sorted(fields)
    tensors = [radii] + [fields[k] for k in sorted(fields)]
    for k, f in zip(names, tensors):
        assert f.shape[:2] == (C, n_local), (k, f.shape)
    _mark(stats, "project", dev)
    row_index, indptr = visible_rows(radii)
    counts = gather_counts(indptr, group)                       # the step's host synchronisation
    _mark(stats, "count", dev)
    plan = plan_exchange(counts, order, owners, rank)
    n_send = int(sum(counts[rank]))
    flat = [f.reshape(C * n_local, -1) for f in tensors]
    widths = [f.shape[1] for f in flat]
    sensor_table = _device_ints(order, torch.int32, dev)
    rows = _PackRows.apply(row_index, n_send, sensor_table, n_local, int(gaussian_start), *flat)
    _mark(stats, "pack", dev)
    received = exchange_rows(rows, plan.send_splits, plan.recv_splits, group)
    _mark(stats, "all_to_all", dev)
    row_map, local_ids = segment_row_map(plan, dev)
    out = _UnpackRows.apply(received, row_map, tuple(widths), tuple(f.dtype == torch.int32 for f in flat))
    _mark(stats, "place", dev)
    sensor_ids, gaussian_ids = out[0], out[1]
    result = {}
    for k, f, o in zip(names, tensors, out[2:]):
        result[k] = o.reshape((o.shape[0],) + tuple(f.shape[2:]))
    if stats is not None:
        row_bytes = 4 * (2 + sum(widths))
        stats.update(row_bytes=row_bytes, rows_sent=n_send, rows_received=plan.src_start[-1],
                     bytes_sent_off_rank=row_bytes * (n_send - plan.send_splits[rank]),
                     bytes_received_off_rank=row_bytes * (plan.src_start[-1] - plan.recv_splits[rank]))
    result["local_sensor_ids"] = local_ids   # per row: index of its sensor among this rank's sensors
    return result, sensor_ids, gaussian_ids, plan


def _mark(stats: Optional[dict], name: str, device) -> None:
    """With ``stats["time"]`` set, records a CUDA event named ``name`` on the current stream into
    ``stats["marks"]``: the stage boundaries a benchmark turns into per-stage times."""
    if stats is not None and stats.get("time"):
        ev = torch.cuda.Event(enable_timing=True)
        ev.record(torch.cuda.current_stream(device))
        stats.setdefault("marks", []).append((name, ev))


def _ordered(t: Optional[Tensor], order: Sequence[int]) -> Optional[Tensor]:
    if t is None or list(order) == list(range(len(order))):
        return t
    return t[_device_ints(order, torch.int64, t.device)]


def rasterization_gaussian_sharded(
    means: Tensor, quats: Tensor, scales: Tensor, opacities: Tensor, colors: Tensor,
    velocities: Optional[Tensor], viewmats: Tensor, Ks: Tensor, width: int, height: int,
    n_gaussians_total: int, gaussian_start: int, linear_velocity: Optional[Tensor] = None,
    angular_velocity: Optional[Tensor] = None, rolling_shutter_time: Optional[Tensor] = None,
    near_plane: float = 0.01, far_plane: float = 1e10, radius_clip: float = 0.0, eps2d: float = 0.3,
    sh_degree: Optional[int] = None, tile_size: int = 16, backgrounds: Optional[Tensor] = None,
    render_mode: str = "RGB", absgrad: bool = False, rasterize_mode: str = "classic",
    owners: Optional[Sequence[int]] = None, group=None, stats: Optional[dict] = None,
):
    """Camera render with the Gaussians split across ranks: the local slice (``means`` etc. are this
    rank's Gaussians, ``gaussian_start`` its first global id, ``colors`` [N_local, D] or SH
    coefficients [N_local, K, 3]) is projected against all C cameras, the visible records travel to
    the camera owners, and each rank composites the cameras it owns. Arguments otherwise as
    ``rasterization`` (gsplat/rendering.py:22-440); ``viewmats`` etc. describe ALL cameras on every rank.

    Returns ``(render_colors [C_local, H, W, X], render_alphas, meta)`` for this rank's cameras in
    ascending global camera order (``meta["sensor_ids"]`` lists them). Gradients flow back to the
    local slice through the mirrored all-to-all.
    """
    from . import ops
    from .rendering import _composite_with_count_check

    world, rank = _world(group)
    C = viewmats.shape[0]
    dev = means.device
    assert render_mode in ("RGB", "D", "ED", "RGB+D", "RGB+ED"), render_mode
    if owners is None:
        owners = sensor_owners(C, world)
    order = sensor_send_order(owners)
    _mark(stats, "start", dev)
    zeros = lambda *s: torch.zeros(*s, device=dev)  # noqa: E731
    viewmats_o, Ks_o = _ordered(viewmats, order), _ordered(Ks, order)
    lin = _ordered(linear_velocity if linear_velocity is not None else zeros(C, 3), order)
    ang = _ordered(angular_velocity if angular_velocity is not None else zeros(C, 3), order)
    rs_all = rolling_shutter_time if rolling_shutter_time is not None else zeros(C)
    rs = _ordered(rs_all, order)
    radii, means2d, depths, conics, comps, pix_vels = ops.fully_fused_projection(
        means, None, quats, scales, velocities, viewmats_o, Ks_o, width, height, lin, ang, rs, eps2d=eps2d,
        near_plane=near_plane, far_plane=far_plane, radius_clip=radius_clip,
        calc_compensations=(rasterize_mode == "antialiased"))
    n_local = means.shape[0]
    opac = opacities[None].expand(C, n_local)
    if comps is not None:
        opac = opac * comps
    with_depth = render_mode in ("RGB+D", "RGB+ED")
    if render_mode in ("D", "ED"):
        cols = depths[..., None]
    elif sh_degree is not None:
        cols = ops.view_dependent_colors(sh_degree, means, ops.camera_centers(viewmats_o), colors, radii,
                                         depths=depths if with_depth else None)
    else:
        cols = colors[None].expand(C, -1, -1) if colors.dim() == 2 else _ordered(colors, order)
        if with_depth:
            cols = torch.cat([cols, depths[..., None]], dim=-1)
    fields = dict(means2d=means2d, depths=depths, conics=conics, opacities=opac.contiguous(), pix_vels=pix_vels,
                  colors=cols.contiguous())
    recv, sensor_ids, gaussian_ids, plan = exchange_projected(fields, radii, gaussian_start, owners, order, group,
                                                              stats)
    mine = plan.mine
    Cl = max(len(mine), 1)
    cam_local = recv["local_sensor_ids"]
    tile_w, tile_h = math.ceil(width / float(tile_size)), math.ceil(height / float(tile_size))
    r_int = recv["radii"]
    opac_r = recv["opacities"].reshape(-1)
    isect = ops.isect_tiles_deferred(recv["means2d"], r_int, recv["depths"].reshape(-1), tile_size, tile_w, tile_h,
                                     packed=True, n_cameras=Cl, camera_ids=cam_local, gaussian_ids=gaussian_ids)
    _mark(stats, "isect", dev)
    mine_t = _device_ints(mine if mine else [0], torch.int64, dev)
    rs_mine = rs_all[mine_t]
    bg = None
    if backgrounds is not None:
        bg = backgrounds[mine_t]
        if with_depth:
            bg = torch.cat([bg, torch.zeros(bg.shape[0], 1, device=dev)], dim=-1)
        elif render_mode in ("D", "ED"):
            bg = torch.zeros(bg.shape[0], 1, device=dev)

    def composite(isect_offsets, flatten_ids, total_follows):
        return ops.rasterize_to_pixels(recv["means2d"], recv["conics"], recv["colors"], opac_r, recv["pix_vels"],
                                       width, height, tile_size, isect_offsets, flatten_ids, rs_mine,
                                       backgrounds=bg, packed=True, absgrad=absgrad, total_follows=total_follows)

    (render_colors, render_alphas), isect_ids, flatten_ids, offsets, tiles_per_gauss = _composite_with_count_check(
        isect, (tile_h, tile_w), composite)
    _mark(stats, "composite", dev)
    if render_mode in ("ED", "RGB+ED"):
        render_colors = torch.cat(
            [render_colors[..., :-1], render_colors[..., -1:] / render_alphas.clamp(min=1e-10)], dim=-1)
    meta = dict(sensor_ids=mine, camera_ids=cam_local, gaussian_ids=gaussian_ids, global_sensor_ids=sensor_ids,
                means2d=recv["means2d"], radii=r_int, depths=recv["depths"].reshape(-1), conics=recv["conics"],
                opacities=opac_r, pix_vels=recv["pix_vels"], tiles_per_gauss=tiles_per_gauss, isect_ids=isect_ids,
                flatten_ids=flatten_ids, isect_offsets=offsets, n_cameras=len(mine), tile_width=tile_w,
                tile_height=tile_h, width=width, height=height, tile_size=tile_size, plan=plan)
    if not mine:
        render_colors, render_alphas = render_colors[:0], render_alphas[:0]
    return render_colors, render_alphas, meta


def lidar_rasterization_gaussian_sharded(
    means: Tensor, quats: Tensor, scales: Tensor, opacities: Tensor, lidar_features: Tensor,
    velocities: Optional[Tensor], viewmats: Tensor, raster_pts: Tensor, tile_elevation_boundaries: Tensor,
    n_gaussians_total: int, gaussian_start: int, linear_velocity: Optional[Tensor] = None,
    angular_velocity: Optional[Tensor] = None, rolling_shutter_time: Optional[Tensor] = None,
    min_azimuth: float = -180, max_azimuth: float = 180, min_elevation: float = -80, max_elevation: float = 80,
    n_elevation_channels: int = 32, azimuth_resolution: float = 0.1, tile_width: int = 32, tile_height: int = 8,
    near_plane: float = 0.01, far_plane: float = 1e10, radius_clip: float = 0.0, eps2d: float = 0.017,
    compute_alpha_sum_until_points: bool = True, compute_alpha_sum_until_points_threshold: float = 0.2,
    absgrad: bool = False, rasterize_mode: str = "classic", use_depth_compensation: bool = True,
    owners: Optional[Sequence[int]] = None, group=None, stats: Optional[dict] = None,
):
    """Lidar render with the Gaussians split across ranks; the lidar twin of
    :func:`rasterization_gaussian_sharded`. ``lidar_features`` is [C, N_local, D] (or [N_local, D],
    shared by all sensors) with D + 1 <= 32, ``viewmats`` / ``raster_pts`` etc. describe ALL C lidars
    on every rank; arguments otherwise as ``lidar_rasterization`` (gsplat/rendering.py:443-819).

    Returns ``(features + range [C_local, H, W, D + 1], alphas, alpha_sum or None, meta)`` for the
    lidars this rank owns, ascending global sensor id (``meta["sensor_ids"]``).
    """
    from . import ops
    from .rendering import _composite_with_count_check

    world, rank = _world(group)
    C = viewmats.shape[0]
    dev = means.device
    n_local = means.shape[0]
    if owners is None:
        owners = sensor_owners(C, world)
    order = sensor_send_order(owners)
    _mark(stats, "start", dev)
    zeros = lambda *s: torch.zeros(*s, device=dev)  # noqa: E731
    lin = _ordered(linear_velocity if linear_velocity is not None else zeros(C, 3), order)
    ang = _ordered(angular_velocity if angular_velocity is not None else zeros(C, 3), order)
    rs = _ordered(rolling_shutter_time if rolling_shutter_time is not None else zeros(C), order)
    radii, means2d, depths, conics, comps, pix_vels, dcomp = ops.fully_fused_lidar_projection(
        means, None, quats, scales, velocities, _ordered(viewmats, order), lin, ang, rs,
        min_elevation=min_elevation, max_elevation=max_elevation, min_azimuth=min_azimuth, max_azimuth=max_azimuth,
        eps2d=eps2d, near_plane=near_plane, far_plane=far_plane, radius_clip=radius_clip,
        calc_compensations=(rasterize_mode == "antialiased"))
    opac = opacities[None].expand(C, n_local)
    if comps is not None:
        opac = opac * comps
    if not use_depth_compensation:
        dcomp = dcomp * 0
    feats = lidar_features[None].expand(C, -1, -1) if lidar_features.dim() == 2 else _ordered(lidar_features, order)
    assert feats.shape[:2] == (C, n_local) and feats.shape[-1] + 1 <= 32, feats.shape
    fields = dict(means2d=means2d, depths=depths, conics=conics, opacities=opac.contiguous(), pix_vels=pix_vels,
                  depth_compensations=dcomp, features=feats.contiguous())
    recv, sensor_ids, gaussian_ids, plan = exchange_projected(fields, radii, gaussian_start, owners, order, group,
                                                              stats)
    mine = plan.mine
    Cl = max(len(mine), 1)
    cam_local = recv["local_sensor_ids"]
    mine_t = _device_ints(mine if mine else [0], torch.int64, dev)
    pts = raster_pts[mine_t].contiguous()
    n_el = math.ceil(n_elevation_channels / tile_height)
    tile_az = azimuth_resolution * tile_width
    n_az = math.ceil((max_azimuth - min_azimuth) / tile_az)
    H, W = pts.shape[1:3]
    depths_r, opac_r = recv["depths"].reshape(-1), recv["opacities"].reshape(-1)
    isect = ops.isect_lidar_tiles_deferred(recv["means2d"], recv["radii"], depths_r, tile_elevation_boundaries,
                                           tile_az, min_azimuth, packed=True, n_cameras=Cl, camera_ids=cam_local,
                                           gaussian_ids=gaussian_ids)
    _mark(stats, "isect", dev)

    def composite(isect_offsets, flatten_ids, total_follows):
        return ops.rasterize_to_points_split(
            recv["means2d"], recv["conics"], recv["features"], depths_r, opac_r, recv["pix_vels"],
            recv["depth_compensations"], pts, W, H, tile_width, tile_height, isect_offsets, flatten_ids,
            compute_alpha_sum_until_points, compute_alpha_sum_until_points_threshold, absgrad=absgrad,
            total_follows=total_follows)

    (feats_r, alphas, alpha_sum, median), isect_ids, flatten_ids, offsets, tiles_per_gauss = (
        _composite_with_count_check(isect, (n_el, n_az), composite))
    _mark(stats, "composite", dev)
    meta = dict(sensor_ids=mine, camera_ids=cam_local, gaussian_ids=gaussian_ids, global_sensor_ids=sensor_ids,
                means2d=recv["means2d"], radii=recv["radii"], depths=depths_r, conics=recv["conics"],
                opacities=opac_r, pix_vels=recv["pix_vels"], tiles_per_gauss=tiles_per_gauss, isect_ids=isect_ids,
                flatten_ids=flatten_ids, isect_offsets=offsets, n_cameras=len(mine), tile_grid_width=n_az,
                tile_grid_height=n_el, width=W, height=H, tile_width=tile_width, tile_height=tile_height,
                median_depths=median, plan=plan)
    if not mine:
        feats_r, alphas, median = feats_r[:0], alphas[:0], median[:0]
        alpha_sum = None if alpha_sum is None else alpha_sum[:0]
        meta["median_depths"] = median
    return feats_r, alphas, alpha_sum, meta


def all_reduce_gradients(params: Sequence[Tensor], group=None) -> None:
    """Sensor-sharded training: sums the parameter gradients of the replicated Gaussians."""
    world, _ = _world(group)
    if world == 1:
        return
    for p in params:
        if p.grad is not None:
            dist.all_reduce(p.grad, op=dist.ReduceOp.SUM, group=group)
