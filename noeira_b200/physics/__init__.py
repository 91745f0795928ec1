from .model import (Actuator, Body, Geom, Joint, Options, RigidModel, half_cheetah, hopper, inverted_double_pendulum,  # noqa: F401
                    pendulum_cart, planar_chain, reacher, walker2d)
