"""Chunked evaluation with host buffers: the rows of a row-sharded evaluation (see shard.py) go through the GPU
chunk by chunk, so that the host-to-device copy of chunk c+1, the kernels of chunk c and the device-to-host copy
of chunk c-1 run at the same time on three streams. With inputs and outputs in pinned host memory a step then
costs about max(upload, download) instead of their sum: PCIe is full duplex.

The graph is recorded once at the chunk's shape; every chunk replays the same compiled program on other device
buffers. Copies are plain cudaMemcpyAsync / cudaMemcpy2DAsync calls (a column slab of a row-major matrix is a
pitched 2-D copy), one per buffer; ordering between the streams is by events. The reference has no device
pipeline of this kind (its backends take host tensors in and hand host tensors back, kurumi_core/src/backend.rs:14-31),
so this file has no counterpart there.
"""
from __future__ import annotations

from dataclasses import dataclass

from cuda.bindings import runtime as cudart

from . import api


def _ok(res):
    err = res[0] if isinstance(res, tuple) else res
    if int(err) != 0:
        raise api.Error(f"CUDA runtime call failed: {err}")
    if isinstance(res, tuple):
        return res[1] if len(res) == 2 else res[1:]
    return None


@dataclass
class HostInput:
    """One graph input in pinned host memory. axis: None = every chunk needs all of it (copied once per step),
    0 = sharded by rows (contiguous slabs), 1 = sharded by columns of a 2-D row-major array (pitched slabs)."""
    node: int
    ptr: int
    shape: tuple
    dtype: int
    axis: int | None


class RowPipeline:
    def __init__(self, gpu: api.CudaBackend, graph: api.Graph, root: int, inputs: list, out_ptr: int, out_rows: int, out_row_bytes: int, chunks: int):
        """`graph` / `root` are recorded at the chunk's shape; `inputs` describe the FULL host arrays; the result has
        `out_rows` rows of `out_row_bytes` bytes (chunk c owns rows [c, c+1) * out_rows / chunks) and is written to `out_ptr`."""
        import numpy as np
        self.gpu, self.graph, self.root, self.inputs, self.chunks = gpu, graph, root, inputs, chunks
        self.out_ptr, self.out_rows, self.out_row_bytes = out_ptr, out_rows, out_row_bytes
        if out_rows % chunks:
            raise api.Error(f"{out_rows} output rows do not split into {chunks} equal chunks")
        self.h2d = _ok(cudart.cudaStreamCreateWithFlags(cudart.cudaStreamNonBlocking))
        self.d2h = _ok(cudart.cudaStreamCreateWithFlags(cudart.cudaStreamNonBlocking))
        self.compute = cudart.cudaStream_t(gpu.stream)
        ev = lambda: _ok(cudart.cudaEventCreateWithFlags(cudart.cudaEventDisableTiming))
        self.ev_in = [ev() for _ in range(chunks)]
        self.ev_k = [ev() for _ in range(chunks)]
        self.ev_rep = ev()
        self.bufs = {}   # node -> [DevTensor, DevTensor] (sharded, double-buffered) or [DevTensor] (replicated)
        for inp in inputs:
            width = api.dtype_width(inp.dtype)
            if inp.axis is None:
                shape = tuple(inp.shape)
            else:
                if inp.shape[inp.axis] % chunks:
                    raise api.Error(f"input axis of {inp.shape[inp.axis]} does not split into {chunks} equal chunks")
                shape = tuple(d // chunks if a == inp.axis else d for a, d in enumerate(inp.shape))
                if inp.axis == 1 and len(inp.shape) != 2:
                    raise api.Error("column sharding needs a 2-D input")
            n = 1 if inp.axis is None else 2
            zeros = np.zeros(int(np.prod(shape)) * width, np.uint8)
            self.bufs[inp.node] = [gpu.upload_ptr(zeros.ctypes.data, zeros.nbytes, shape, inp.dtype) for _ in range(n)]

    def _copy_in(self, inp: HostInput, c: int, dst: api.DevTensor):
        width = api.dtype_width(inp.dtype)
        kind = cudart.cudaMemcpyKind.cudaMemcpyHostToDevice
        if inp.axis is None:
            _ok(cudart.cudaMemcpyAsync(dst.ptr, inp.ptr, dst.nbytes, kind, self.h2d))
        elif inp.axis == 0:
            _ok(cudart.cudaMemcpyAsync(dst.ptr, inp.ptr + c * dst.nbytes, dst.nbytes, kind, self.h2d))
        else:
            rows, cols = inp.shape
            w = cols // self.chunks * width
            _ok(cudart.cudaMemcpy2DAsync(dst.ptr, w, inp.ptr + c * w, cols * width, w, rows, kind, self.h2d))

    def step(self):
        """One evaluation of the whole problem, host buffers in, host buffer out; returns after the result is in host memory."""
        gpu = self.gpu
        for inp in self.inputs:
            if inp.axis is None:
                self._copy_in(inp, 0, self.bufs[inp.node][0])
        _ok(cudart.cudaEventRecord(self.ev_rep, self.h2d))
        _ok(cudart.cudaStreamWaitEvent(self.compute, self.ev_rep, 0))
        outs = []
        chunk_bytes = self.out_rows // self.chunks * self.out_row_bytes
        for c in range(self.chunks):
            b = c & 1
            if c >= 2:   # the kernels of chunk c - 2 read this buffer
                _ok(cudart.cudaStreamWaitEvent(self.h2d, self.ev_k[c - 2], 0))
            feeds = {}
            for inp in self.inputs:
                if inp.axis is None:
                    feeds[inp.node] = self.bufs[inp.node][0]
                else:
                    self._copy_in(inp, c, self.bufs[inp.node][b])
                    feeds[inp.node] = self.bufs[inp.node][b]
            _ok(cudart.cudaEventRecord(self.ev_in[c], self.h2d))
            _ok(cudart.cudaStreamWaitEvent(self.compute, self.ev_in[c], 0))
            out = gpu.eval_device(self.graph, [self.root], None, feeds)[0]
            _ok(cudart.cudaEventRecord(self.ev_k[c], self.compute))
            _ok(cudart.cudaStreamWaitEvent(self.d2h, self.ev_k[c], 0))
            if out.nbytes != chunk_bytes:
                raise api.Error(f"chunk result has {out.nbytes} bytes, expected {chunk_bytes}")
            _ok(cudart.cudaMemcpyAsync(self.out_ptr + c * chunk_bytes, out.ptr, chunk_bytes, cudart.cudaMemcpyKind.cudaMemcpyDeviceToHost, self.d2h))
            outs.append(out)   # its memory goes back to the pool only after the copy out has finished
        _ok(cudart.cudaStreamSynchronize(self.d2h))
        for o in outs:
            o.free()

    def close(self):
        for bufs in self.bufs.values():
            for b in bufs:
                b.free()
        self.bufs = {}
        for e in self.ev_in + self.ev_k + [self.ev_rep]:
            cudart.cudaEventDestroy(e)
        cudart.cudaStreamDestroy(self.h2d)
        cudart.cudaStreamDestroy(self.d2h)
