"""Command line privacy calculator for DP-SGD.

    python -m opacus_b200.scripts.compute_dp_sgd_privacy -r 0.04 -n 1.5 -e 90 [-d 1e-5] [-a 1.5 2 4 8 16 32]

prints the (epsilon, delta) guarantee of ``epochs / sample_rate`` steps of the
Poisson-subsampled Gaussian mechanism under RDP accounting, and the optimal
order.  Same flags as ``opacus/scripts/compute_dp_sgd_privacy.py:142-195``.
"""
import argparse
import math
from typing import List, Optional, Tuple

from ..accountants.analysis import rdp as privacy_analysis
from ..accountants.rdp import RDPAccountant


def _apply_dp_sgd_analysis(*, sample_rate: float, noise_multiplier: float, steps: int,
                           alphas: List[float], delta: float, verbose: bool = True) -> Tuple[float, float]:
    rdp = privacy_analysis.compute_rdp(q=sample_rate, noise_multiplier=noise_multiplier, steps=steps, orders=alphas)
    eps, opt_alpha = privacy_analysis.get_privacy_spent(orders=alphas, rdp=rdp, delta=delta)
    if verbose:
        print(f"DP-SGD with\n\tsampling rate = {100 * sample_rate:.3g}%,\n\tnoise_multiplier = {noise_multiplier},"
              f"\n\titerated over {steps} steps,\nsatisfies differential privacy with\n\tepsilon = {eps:.3g},"
              f"\n\tdelta = {delta}.\nThe optimal alpha is {opt_alpha}.")
        if opt_alpha == max(alphas) or opt_alpha == min(alphas):
            print("The privacy estimate is likely to be improved by expanding the set of alpha orders.")
    return float(eps), float(opt_alpha)


def compute_dp_sgd_privacy(*, sample_rate: float, noise_multiplier: float, epochs: int, delta: float,
                           alphas: Optional[List[float]] = None, verbose: bool = True) -> Tuple[float, float]:
    """(epsilon, optimal order) after ``epochs`` epochs."""
    if sample_rate > 1:
        raise ValueError("sample_rate must be no greater than 1")
    steps = int(math.ceil(epochs / sample_rate))
    return _apply_dp_sgd_analysis(sample_rate=sample_rate, noise_multiplier=noise_multiplier, steps=steps,
                                  alphas=alphas or RDPAccountant.DEFAULT_ALPHAS, delta=delta, verbose=verbose)


def main(argv=None):
    ap = argparse.ArgumentParser(description="RDP privacy calculator for DP-SGD")
    ap.add_argument("-r", "--sample-rate", type=float, required=True, help="batch size / dataset size")
    ap.add_argument("-n", "--noise-multiplier", type=float, required=True, help="noise std / clipping norm")
    ap.add_argument("-e", "--epochs", type=int, required=True)
    ap.add_argument("-d", "--delta", type=float, default=1e-5)
    ap.add_argument("-a", "--alphas", type=float, nargs="+", default=RDPAccountant.DEFAULT_ALPHAS)
    args = ap.parse_args(argv)
    compute_dp_sgd_privacy(sample_rate=args.sample_rate, noise_multiplier=args.noise_multiplier,
                           epochs=args.epochs, delta=args.delta, alphas=args.alphas)


if __name__ == "__main__":
    main()
