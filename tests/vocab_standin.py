"""A CPU stand-in for the two vocab-sharding kernels, speaking the same record format
(include/gorch_cuda_shim.h: 16 header bytes + 128 pairs of (f32 bits, u32 index)). It answers
from the CPU oracle and exists only so that the host-side exchange can be tested without a GPU."""
import numpy as np

VS_CAND = 128
REC = 16 + 8 * VS_CAND


def bf16_to_f32(a):
    return (a.astype(np.uint32) << 16).view(np.float32)


class StandInSampler:
    def vocab_local(self, logits_slice, cfgs, col_offset):
        x = bf16_to_f32(logits_slice) if logits_slice.dtype == np.uint16 else np.asarray(logits_slice, np.float32)
        B, Vs = x.shape
        rec = np.zeros((B, REC), dtype=np.uint8)
        for b in range(B):
            k = int(cfgs["top_k"][b])
            T = float(cfgs["temperature"][b])
            row = x[b]
            hdr = rec[b, :16].view(np.uint32)
            if T == 0.0:
                i = int(np.argmax(row))                    # first maximum
                hdr[0] = row[i:i + 1].view(np.uint32)[0]; hdr[1] = 1
                pairs = rec[b, 16:].view(np.uint32).reshape(VS_CAND, 2)
                pairs[0] = (row[i:i + 1].view(np.uint32)[0], i + col_offset)
                continue
            if not (0 < k <= VS_CAND):
                hdr[2] = 8                                 # VS_UNSUPPORTED
                continue
            kk = min(k, Vs)
            tau = np.sort(row)[::-1][kk - 1]
            idx = np.nonzero(row >= tau)[0]
            if len(idx) > VS_CAND:
                hdr[2] = 4                                 # VS_OVERFLOW
                continue
            hdr[0] = np.float32(row.max()).reshape(1).view(np.uint32)[0]
            hdr[1] = len(idx)
            pairs = rec[b, 16:].view(np.uint32).reshape(VS_CAND, 2)
            pairs[:len(idx), 0] = row[idx].view(np.uint32)
            pairs[:len(idx), 1] = idx + col_offset
        return rec

    def vocab_merge(self, all_records, cfgs, uniforms, V):
        from oracle import oracle as orc
        nranks, B = all_records.shape[:2]
        ids = np.full(B, -1, np.int32)
        flags = np.zeros(B, np.uint32)
        for b in range(B):
            row = np.full(V, -np.inf, np.float32)
            bad = False
            for r in range(nranks):
                hdr = all_records[r, b, :16].view(np.uint32)
                if hdr[2] != 0:
                    bad = True
                n = int(hdr[1])
                pairs = all_records[r, b, 16:].view(np.uint32).reshape(VS_CAND, 2)
                row[pairs[:n, 1].astype(np.int64)] = pairs[:n, 0].copy().view(np.float32)
            if bad:
                flags[b] = 0x80
                continue
            res = orc.sample_batch(row[None], cfgs[b:b + 1], uniforms[b:b + 1], want_info=False, flags=orc.FAST_KTH)
            ids[b] = res["ids"][0]
        return ids, flags
