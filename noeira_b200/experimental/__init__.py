"""Research prototypes next to the main packages: the eager tape mode of ``nn`` (``functional``), a predictive-coding
network (``pcn``), a JEPA-style latent world model (``jepa``) and the sheaf world model with holonomy as an observable
(``swm``).  Reference: noeira/experimental/."""
