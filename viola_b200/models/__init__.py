"""Model zoo: the DiT family used by the reference experiments and the headline benchmark."""

from .dit import DiT, NoiseSchedule, diffusion_loss, muon_parameter_groups

__all__ = ["DiT", "NoiseSchedule", "diffusion_loss", "muon_parameter_groups"]
