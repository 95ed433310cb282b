from .sampler import Sampler, uniform_for
