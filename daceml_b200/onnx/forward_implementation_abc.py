"""The implementation registry of the ONNX library nodes.

Same contract as the reference's ``ONNXForward`` (``daceml/onnx/forward_implementation_abc.py:12-55``):
a class with static ``forward_can_be_applied(node, state, sdfg) -> bool`` and
``forward(node, state, sdfg)``, registered under an ONNX op name and an implementation name.
The reference turns the ABC into a registry with ``dace.registry.make_registry``; the two methods
that decorator adds (``register`` / ``extensions``) are written out here.
"""
import abc
import typing


class ONNXForward(abc.ABC):
    """ ABC for ONNX op forward implementations.

        The register function expects an argument `op` containing the ONNX op name (string).
    """
    _registry_: typing.Dict[type, dict] = {}

    @classmethod
    def register(cls, subclass, **kwargs):
        cls._registry_[subclass] = kwargs

    @classmethod
    def unregister(cls, subclass):
        cls._registry_.pop(subclass, None)

    @classmethod
    def extensions(cls):
        return cls._registry_

    @staticmethod
    def forward_can_be_applied(node, state, sdfg) -> bool:
        """ Return whether this expansion can be applied.

            :param node: the candidate node.
            :param state: the candidate state.
            :param sdfg: the candidate sdfg.
            :return: whether this expansion can be applied.
        """
        return True

    @staticmethod
    @abc.abstractmethod
    def forward(node, state, sdfg):
        """ Expand `node` and return its expansion.

            :param node: the candidate node.
            :param state: the candidate state.
            :param sdfg: the candidate sdfg.
            :return: the expanded node.
        """
        ...

    @classmethod
    def registered_implementations(cls, op_name: str) -> typing.List[typing.Tuple[str, "ONNXForward"]]:
        impls = []
        for impl, args in cls.extensions().items():
            if "op" in args and args["op"] == op_name:
                impls.append((args["name"], impl))
        return impls
