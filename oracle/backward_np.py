"""TEST INFRASTRUCTURE: numpy restatement (float64 accumulation) of the reference's GRU backward
pass: kernel::PointwiseOperations + BackwardPass<T>::Run (src/gru_backward_gpu.cu:26-88, 240-292)
and, with masks, PointwiseOperationsQuant + BackwardPassQuant<T>::Run
(src/gru_backward_gpu_quant.cu:72-250, 380-490), zoneout off.

The reference's GEMMs are cuBLAS SGEMMs and its bias gradients are atomicAdd sums, both of
unspecified summation order; here every sum is accumulated in float64, the most accurate answer,
so that any correct fp32 implementation lies within a few 1e-6 relative.  Parity of this file
is pinned on the GPU box against the reference's own GPU backward
(tests/test_gpu_vs_reference_gpu.py) and on the CPU against torch autograd through torch.nn.GRU
(tests/test_backward_oracle.py)."""
import numpy as np

MASK_NAMES = ("x", "h0", "W", "R", "bw", "br", "ih_linear", "hh_linear", "gate_input", "gate_output", "h")


def gru_backward(W, R, x, dh_new, h, v, masks=None, dh_last=None):
    """W [I,3H], R [H,3H] (haste layout, gates z, r, g), x [T,B,I], dh_new / h [(T+1),B,H],
    v [T,B,4H] = (z, r, g, R*h_g + br_g).  masks: dict name -> uint8 array (1 keeps the gradient).
    Returns (dx [T,B,I], dW, dR, dbw, dbr, dh [B,H]) as float32."""
    masks = masks or {}
    T, B, I = x.shape
    H = R.shape[0]
    f8 = np.float64

    def m(name, shape):
        a = masks.get(name)
        return None if a is None else np.asarray(a, f8).reshape(shape)

    m_hh, m_gin, m_gout = m("hh_linear", (T, B, 3 * H)), m("gate_input", (T, B, 3 * H)), m("gate_output", (T, B, 3 * H))
    m_h = m("h", (T, B, H))
    dh = np.zeros((B, H), f8) if dh_last is None else np.asarray(dh_last, f8).copy()
    dp = np.zeros((T, B, 3 * H), f8)
    dq = np.zeros((T, B, 3 * H), f8)
    Rt = np.asarray(R, f8).T                       # [3H, H]
    for i in range(T - 1, -1, -1):
        dh_total = np.asarray(dh_new[i + 1], f8) + dh
        if m_h is not None:
            dh_total = dh_total * m_h[i]
        z, r, g, q_g = (np.asarray(v[i][:, k * H:(k + 1) * H], f8) for k in range(4))
        dh = z * dh_total
        dg = (1.0 - z) * dh_total
        dz = (np.asarray(h[i], f8) - g) * dh_total
        dp_g = (1.0 - g * g) * dg
        dq_g = dp_g * r
        dr = dp_g * q_g
        dp_r = r * (1.0 - r) * dr
        dp_z = z * (1.0 - z) * dz
        p = np.concatenate([dp_z, dp_r, dp_g], 1)
        q = np.concatenate([dp_z, dp_r, dq_g], 1)
        for mk in (m_gout, m_gin):
            if mk is not None:
                p, q = p * mk[i], q * mk[i]
        if m_hh is not None:
            q = q * m_hh[i]
        dp[i], dq[i] = p, q
        dh = dh + q @ Rt
    dbw = dp.sum((0, 1))
    dbr = dq.sum((0, 1))
    if masks.get("bw") is not None:
        dbw = dbw * np.asarray(masks["bw"], f8)
    if masks.get("br") is not None:
        dbr = dbr * np.asarray(masks["br"], f8)
    if masks.get("ih_linear") is not None:
        dp = dp * m("ih_linear", (T, B, 3 * H))
    dx = dp @ np.asarray(W, f8).T
    if masks.get("x") is not None:
        dx = dx * m("x", (T, B, I))
    dR = np.asarray(h[:T], f8).reshape(T * B, H).T @ dq.reshape(T * B, 3 * H)
    if masks.get("R") is not None:
        dR = dR * m("R", (H, 3 * H))
    dW = np.asarray(x, f8).reshape(T * B, I).T @ dp.reshape(T * B, 3 * H)
    if masks.get("W") is not None:
        dW = dW * m("W", (I, 3 * H))
    if masks.get("h0") is not None:
        dh = dh * m("h0", (B, H))
    return tuple(a.astype(np.float32) for a in (dx, dW, dR, dbw, dbr, dh))
