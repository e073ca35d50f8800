"""Generate the golden fixtures in this directory by running the UNMODIFIED reference.

Run once, in a container where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's own PyTorch model (train/train_general_ring_no_gain.py:21-137, the
twin of what the CUDA operator computes), its losses (train/train_ring_attractor.py:190-220,
:275-298), its initial-bump helper (:21-52) and its input generator
(utils/generate_av_integration_data.py:11-58), runs them on seeded inputs on CPU in fp32 and
stores inputs and outputs as small .npz files.  matplotlib is stubbed when absent (the
reference imports it at module top but the functions used here never touch it).
The tests only read the .npz files; they never need the reference checkout.
"""
import os
import sys
import types

import numpy as np
import torch


def import_reference(root):
    try:
        import matplotlib.pyplot  # noqa: F401
    except Exception:
        mpl = types.ModuleType("matplotlib")
        plt = types.ModuleType("matplotlib.pyplot")
        mpl.pyplot = plt
        sys.modules["matplotlib"] = mpl
        sys.modules["matplotlib.pyplot"] = plt
    sys.path.insert(0, root)
    sys.path.insert(0, os.path.join(root, "train"))  # first: the root holds a same-named CUDA-only script
    import train_general_ring_no_gain as m_nogain  # the file under train/
    import train_ring_attractor as m_ring
    from utils import generate_av_integration_data as m_data
    return m_nogain, m_ring, m_data


def model_case(m_nogain, m_ring, m_data, name, N, B, T, act, a_dim, seed):
    """Reference model at its native constants (alpha=0.15, randn/sqrt(N) weights, Gaussian bump)."""
    torch.manual_seed(seed)
    model = m_nogain.GeneralizedRingAttractorNoGain(N, action_dim=a_dim, activation=act, initialization="random")
    av, angle = m_data.generate_av_integration_data_ultra_fast(B, T)
    A = torch.zeros(B, T, a_dim)
    A[:, :, 0] = torch.relu(-av)
    A[:, :, 1] = torch.relu(av)
    if a_dim > 2:  # exercise the generic action path too
        A[:, :, 2:] = 0.05 * torch.rand(B, T, a_dim - 2)
    r_init = m_ring.create_initial_bump(angle[:, 0], N)
    wave, bump = model(A, r_init=r_init)
    loss_cos = m_ring.cosine_similarity_loss(wave, angle)
    loss_amp = m_ring.bump_amplitude_loss(bump)
    total = loss_cos + 0.2 * loss_amp
    total.backward(retain_graph=True)
    out = dict(N=N, B=B, T=T, a_dim=a_dim, act=act, alpha=0.15, J0=-0.1, J1=0.1,
               av=av, angle=angle, A=A, r_init=r_init, Wo=model.Wo.detach(), Wa=model.Wa.detach(),
               wave=wave.detach(), bump=bump.detach(), loss_cos=loss_cos.detach(), loss_amp=loss_amp.detach(),
               loss=total.detach(), dWo=model.Wo.grad.clone(), dWa=model.Wa.grad.clone(),
               decoded=m_ring.decode_angle_from_population_vector(wave.detach()))
    # gradient of a plain sum-of-history loss w.r.t. a random cotangent: pins the BPTT alone
    model.zero_grad()
    cot = torch.randn(B, T, N)
    (bump * cot).sum().backward()
    out.update(cot=cot, dWo_cot=model.Wo.grad.clone(), dWa_cot=model.Wa.grad.clone())
    np.savez_compressed(os.path.join(os.path.dirname(__file__), name + ".npz"),
                        **{k: (v.numpy() if torch.is_tensor(v) else np.asarray(v)) for k, v in out.items()})
    print(name, "loss", float(total.detach()))


def generator_case(m_data, name, B, T, seed, max_av):
    torch.manual_seed(seed)
    av, angle = m_data.generate_av_integration_data_ultra_fast(B, T, 0.1, [0.2, 0.5, 0.8], max_av)
    np.savez_compressed(os.path.join(os.path.dirname(__file__), name + ".npz"),
                        B=B, T=T, seed=seed, max_av=max_av, av=av.numpy(), angle=angle.numpy())
    print(name, "av nonzero frac", float((av != 0).float().mean()))


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/reference")
    ref = sys.argv[1]
    m_nogain, m_ring, m_data = import_reference(ref)
    model_case(m_nogain, m_ring, m_data, "ref_tanh_n24", 24, 5, 12, "tanh", 2, 1)
    model_case(m_nogain, m_ring, m_data, "ref_relu_n40", 40, 6, 9, "relu", 2, 2)
    model_case(m_nogain, m_ring, m_data, "ref_gelu_n32_a4", 32, 4, 10, "gelu", 4, 3)
    model_case(m_nogain, m_ring, m_data, "ref_gelu_n120", 120, 4, 8, "gelu", 2, 4)
    generator_case(m_data, "ref_generator", 16, 40, 7, 0.1 * np.pi)
    generator_case(m_data, "ref_generator_slow", 8, 50, 8, 0.05 * np.pi)
