"""Whole-model weight quantization and per-layer NVFP4 GEMMs for a Llama-3-8B-shaped linear stack.

32 decoder layers, each with q 4096x4096, k/v 1024x4096, o 4096x4096, gate/up 14336x4096 and down 4096x14336
(rows = output features N, columns = input features K).  Weights are random bf16 N(0, 0.02); the importance of a
weight's input channels is the squared norm of synthetic N(0,1) calibration activations [2048, K] (K = 4096, or
14336 for `down`, whose input is the MLP's hidden activation).  Layers are partitioned contiguously across ranks
(4 per GPU on 8 GPUs); nothing is communicated while quantizing, and each layer's GEMMs run where the layer lives.

  python -m nvfp4quant_test_b200.llama_stack --layers 32 --batches 1 32 256 4096
  python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m nvfp4quant_test_b200.llama_stack

Prints one JSON line per rank-0 run with per-phase device times (CUDA events, max over ranks).
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from . import helper as H
from . import kernels as K

# name -> (N = out features, K = in features)
LAYER_SHAPES = {
    "q": (4096, 4096), "k": (1024, 4096), "v": (1024, 4096), "o": (4096, 4096),
    "gate": (14336, 4096), "up": (14336, 4096), "down": (4096, 14336),
}
CALIB_ROWS = 2048


def layers_for_rank(n_layers: int, rank: int, world: int) -> range:
    """Contiguous block of layers owned by `rank`; sizes differ by at most one."""
    base, extra = divmod(n_layers, world)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


def weights_per_layer() -> int:
    return sum(n * k for n, k in LAYER_SHAPES.values())


def make_layer(layer: int, device, seed: int = 0) -> dict[str, torch.Tensor]:
    gen = torch.Generator(device=device)
    gen.manual_seed(seed * 100003 + layer)
    return {name: torch.normal(0.0, 0.02, size=shape, generator=gen, device=device, dtype=torch.bfloat16)
            for name, shape in LAYER_SHAPES.items()}


def make_calibration(device, seed: int = 0) -> dict[int, torch.Tensor]:
    """One activation batch per distinct input width, shared by all layers."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed + 7)
    return {k: torch.normal(0.0, 1.0, size=(CALIB_ROWS, k), generator=gen, device=device, dtype=torch.bfloat16)
            for k in sorted({k for _, k in LAYER_SHAPES.values()})}


def quantize_weight(w: torch.Tensor, importance: torch.Tensor, fp8_max: float = H.FP8_E4M3_MAX_4OVER6):
    """(codes, swizzled scales, global_scale) with the importance-weighted ScaleSweep quantizer."""
    gs, gs_inv = H.get_nvfp4_global_scale(w, fp8_max)
    codes, scales = K.scalesweep_weighted_mse_nvfp4_quant_impl(w, importance, gs_inv)
    return codes, scales, gs


def quantize_layer(weights: dict[str, torch.Tensor], importance: dict[int, torch.Tensor], buffers: dict | None = None):
    """{name: (codes, scales, global_scale)}.  With `buffers` ({name: (codes, scales)} from `allocate_layer`) the
    quantizer writes into them through the `_out` entry point, as a loader that owns its weight storage would."""
    if buffers is None:
        return {name: quantize_weight(w, importance[w.shape[1]]) for name, w in weights.items()}
    out = {}
    for name, w in weights.items():
        codes, scales = buffers[name]
        gs, gs_inv = H.get_nvfp4_global_scale(w, H.FP8_E4M3_MAX_4OVER6)
        K.scalesweep_weighted_mse_nvfp4_quant_out(w, importance[w.shape[1]], gs_inv, True, output=codes, output_scale=scales)
        out[name] = (codes, scales.view(torch.float8_e4m3fn), gs)
    return out


def allocate_layer(device) -> dict[str, tuple[torch.Tensor, torch.Tensor]]:
    """Output storage of one quantized layer (codes + tiled scales per matrix)."""
    return {name: K.create_fp4_output_tensors(n, k, device, True) for name, (n, k) in LAYER_SHAPES.items()}


def stack_weight_scales(qlayer: dict) -> dict[int, tuple[torch.Tensor, dict[str, int]]]:
    """{K: (fp32 vector of the global scales of the layer's matrices with K input features, {name: slot})}.
    Built once per layer so that a forward pass needs one multiplication per input width for all its alphas."""
    by_k: dict[int, list[str]] = {}
    for name, (codes, _, _) in qlayer.items():
        by_k.setdefault(codes.shape[1] * 2, []).append(name)
    return {k: (torch.stack([qlayer[n][2].reshape(()).float() for n in names]), {n: i for i, n in enumerate(names)})
            for k, names in by_k.items()}


def prepare_layer(qlayer: dict) -> dict:
    """{name: PreparedWeight} for a quantized layer: the weights' tensor maps are encoded once, not per GEMM call."""
    return {name: K.PreparedWeight(codes, scales) for name, (codes, scales, _) in qlayer.items()}


# matrices that read the same activation in a decoder layer (q / k / v the normed hidden state, gate / up the normed
# post-attention state); o and down have inputs of their own
WEIGHT_GROUPS = (("q", "k", "v"), ("o",), ("gate", "up"), ("down",))
GROUPED_MAX_TOKENS = 64    # beyond, the per-matrix kernels on forked streams are faster (96 tokens: 1.95 against 2.05 ms)


def layer_gemms_grouped(qlayer: dict, acts: dict[int, torch.Tensor], weight_scales: dict, prepared: dict):
    """The layer's GEMMs at a decode-sized batch, on the current stream: per input width one global scale and one
    unweighted sweep of the activation, then one grouped launch per WEIGHT_GROUPS entry (the output scale = activation
    global scale x weight global scale is formed inside the kernel).  Every launch is a programmatic dependent launch
    of the one before it.  Returns {name: bf16 [tokens, N]}."""
    out = {}
    qact: dict[int, tuple] = {}
    for group in WEIGHT_GROUPS:
        k = qlayer[group[0]][0].shape[1] * 2
        if k not in qact:
            x = acts[k]
            gs_x, gs_x_inv = H.get_nvfp4_global_scale(x, H.FP8_E4M3_MAX_4OVER6)
            qa, sa = K.scalesweep_mse_nvfp4_quant_impl(x, gs_x_inv)
            qact[k] = (qa, sa, gs_x.reshape(1))
        qa, sa, gs_x = qact[k]
        vec, slots = weight_scales[k]
        ys = K.nvfp4_scaled_mm_grouped(qa, sa, gs_x, [prepared[n] for n in group],
                                       [vec[slots[n]:slots[n] + 1] for n in group])
        out.update(zip(group, ys))
    return out


class DecodeLayer:
    """layer_gemms_grouped with everything that does not depend on the activations done once: buffers allocated,
    arguments checked, argument arrays built (kernels.ActivationQuantizer / kernels.LinearGroup).  A call is two
    quantizer calls and four grouped GEMM calls into the C ABI, which is what lets a decode step be launched eagerly at
    about the speed of a CUDA-graph replay.  Outputs are overwritten by the next call."""

    def __init__(self, qlayer: dict, weight_scales: dict, prepared: dict, tokens: int, device):
        self.quantizers = {}
        self.groups = []
        for group in WEIGHT_GROUPS:
            k = qlayer[group[0]][0].shape[1] * 2
            if k not in self.quantizers:
                self.quantizers[k] = K.ActivationQuantizer(tokens, k, device)
            vec, slots = weight_scales[k]
            self.groups.append((group, k, K.LinearGroup([prepared[n] for n in group],
                                                        [vec[slots[n]:slots[n] + 1] for n in group], tokens)))

    def __call__(self, acts: dict[int, torch.Tensor]) -> dict[str, torch.Tensor]:
        quantized = {k: q(acts[k]) for k, q in self.quantizers.items()}
        out = {}
        for group, k, linear in self.groups:
            codes, scales, gs = quantized[k]
            out.update(zip(group, linear(codes, scales, gs)))
        return out


def layer_gemms(qlayer: dict, acts: dict[int, torch.Tensor], act_importance: dict[str, torch.Tensor],
                weight_scales: dict | None = None, side_streams: list | None = None, prepared: dict | None = None):
    """y = x @ W.T for every matrix of the layer with NVFP4 operands; activations quantized with the unweighted sweep
    unless an importance vector for them is given.  Returns {name: bf16 [tokens, N]}.

    The GEMMs of a layer are independent of one another.  With `side_streams` they are dealt out over those streams
    (forked from and joined back into the current stream, which also works under CUDA-graph capture), so that at
    small token counts, where one GEMM does not fill the GPU, several run at the same time."""
    if weight_scales is None:
        weight_scales = stack_weight_scales(qlayer)
    main = torch.cuda.current_stream()
    out = {}
    qact: dict[int, tuple] = {}
    used = []
    for i, (name, (codes, scales, gs_w)) in enumerate(qlayer.items()):
        k = codes.shape[1] * 2
        if k not in qact:
            x = acts[k]
            gs_x, gs_x_inv = H.get_nvfp4_global_scale(x, H.FP8_E4M3_MAX_4OVER6)
            imp = act_importance.get(name)
            if imp is None:
                qa, sa = K.scalesweep_mse_nvfp4_quant_impl(x, gs_x_inv)
            else:
                qa, sa = K.scalesweep_weighted_mse_nvfp4_quant_impl(x, imp, gs_x_inv)
            ready = None
            if side_streams:
                ready = torch.cuda.Event()
                alphas = gs_x.float() * weight_scales[k][0]
                ready.record(main)
            else:
                alphas = gs_x.float() * weight_scales[k][0]      # alphas of every matrix fed by this input
            qact[k] = (qa, sa, alphas, ready)
        qa, sa, alphas, ready = qact[k]
        slot = weight_scales[k][1][name]
        def mm():
            if prepared is not None:
                return K.nvfp4_scaled_mm_prepared(qa, sa, alphas[slot:slot + 1], prepared[name])
            return K.nvfp4_scaled_mm(qa, codes, sa, scales, alphas[slot:slot + 1], torch.bfloat16)

        if side_streams:
            st = side_streams[i % len(side_streams)]
            st.wait_event(ready)
            with torch.cuda.stream(st):
                out[name] = mm()
            if st not in used:
                used.append(st)
        else:
            out[name] = mm()
    for st in used:
        done = torch.cuda.Event()
        done.record(st)
        main.wait_event(done)
    return out


def run(n_layers: int, token_batches: list[int], seed: int = 0, use_graph: bool = True, n_streams: int = 4,
        progress=None) -> dict:
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    own_group = world > 1 and not dist.is_initialized()
    if own_group:
        if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
            os.environ["NCCL_DEBUG"] = "WARN"      # keep stdout to the JSON line
        dist.init_process_group("nccl", device_id=dev)

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_ms(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    note = progress or (lambda _msg: None)
    mine = layers_for_rank(n_layers, rank, world)
    calib = make_calibration(dev, seed)
    importance = {k: H.channel_square_norm(x) for k, x in calib.items()}
    layers = [make_layer(i, dev, seed) for i in mine]
    # warm-up (first launches pay module loading), then the timed quantization of all owned layers
    if layers:
        quantize_weight(layers[0]["k"], importance[4096])
    sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # weight storage is allocated up front (cudaMalloc of fresh blocks is not what is being measured)
    buffers = [allocate_layer(dev) for _ in layers]
    sync()
    note("quantizing")
    e0.record()
    qlayers = [quantize_layer(w, importance, b) for w, b in zip(layers, buffers)]
    e1.record()
    sync()
    first_pass_ms = max_ms(e0.elapsed_time(e1))
    # second pass into the same storage: the first one also pays for whatever the caching allocator has to fetch from
    # the driver for its small temporaries (tens of milliseconds after an empty_cache), which is not quantization time
    e0.record()
    qlayers = [quantize_layer(w, importance, b) for w, b in zip(layers, buffers)]
    e1.record()
    sync()
    wscales = [stack_weight_scales(q) for q in qlayers]
    prepared = [prepare_layer(q) for q in qlayers]
    side = [torch.cuda.Stream(device=dev) for _ in range(n_streams)] if n_streams > 1 else None
    quant_ms = max_ms(e0.elapsed_time(e1))
    n_weights = n_layers * weights_per_layer()
    result = {
        "layers": n_layers, "n_gpus": world, "weights": n_weights,
        "quantize_ms": quant_ms, "quantize_first_pass_ms": first_pass_ms,
        "quantize_gweights_per_s": n_weights / (quant_ms * 1e-3) / 1e9,
        "gemm": [],
    }
    for tokens in token_batches:
        gen = torch.Generator(device=dev)
        gen.manual_seed(seed + 1000 + tokens)
        acts = {k: torch.normal(0.0, 1.0, size=(tokens, k), generator=gen, device=dev, dtype=torch.bfloat16)
                for k in calib}
        grouped = tokens <= GROUPED_MAX_TOKENS
        decode = [DecodeLayer(q, ws, pw, tokens, dev) for q, ws, pw in zip(qlayers, wscales, prepared)] if grouped else None

        def all_layers():
            if grouped:
                for layer in decode:
                    layer(acts)
            else:
                for q, ws, pw in zip(qlayers, wscales, prepared):
                    layer_gemms(q, acts, {}, ws, side, pw)

        note(f"tokens {tokens}: eager pass")
        all_layers()
        sync()
        # the same pass launched eagerly, timed from the host's first call to the GPU's last kernel (steady state: the
        # faster of two passes, the first one still pays one-time costs of the first launches of a kernel)
        eager_ms = float("inf")
        for _ in range(2):
            e0.record()
            all_layers()
            e1.record()
            sync()
            eager_ms = min(eager_ms, max_ms(e0.elapsed_time(e1)))
        graph = None
        if use_graph and qlayers:
            # every launch is asynchronous and allocation-free at the C ABI, so the whole per-rank layer stack
            # records into one CUDA graph; replaying it removes the per-launch host cost that dominates small batches
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                all_layers()
            note(f"tokens {tokens}: first replay")
            graph.replay()
            sync()
        note(f"tokens {tokens}: timed replay")
        e0.record()
        if graph is not None:
            graph.replay()
        else:
            all_layers()
        e1.record()
        sync()
        ms = max_ms(e0.elapsed_time(e1))
        flops = 2.0 * tokens * weights_per_layer() * n_layers
        result["gemm"].append({"tokens": tokens, "ms_all_layers": ms, "eager_ms_all_layers": eager_ms,
                               "tflops": flops / (ms * 1e-3) / 1e12,
                               "cuda_graph": graph is not None, "streams": 1 if grouped else n_streams,
                               "launches": "grouped (q+k+v, o, gate+up, down), one stream" if grouped else "one per matrix",
                               "includes": "activation global scale + quantization + 7 GEMMs per layer"})
    if own_group:
        dist.destroy_process_group()
    return result if rank == 0 else {}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--batches", type=int, nargs="*", default=[1, 32, 256, 4096])
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--streams", type=int, default=4,
                    help="streams the GEMMs of a layer are dealt out over (1 = all on the current stream)")
    ap.add_argument("--no-graph", action="store_true", help="launch the GEMM phase eagerly instead of replaying a CUDA graph")
    args = ap.parse_args()
    res = run(args.layers, args.batches, args.seed, use_graph=not args.no_graph, n_streams=args.streams)
    if res:
        print(json.dumps(res))


if __name__ == "__main__":
    main()
