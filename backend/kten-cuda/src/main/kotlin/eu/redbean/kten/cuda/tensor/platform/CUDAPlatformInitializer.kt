package eu.redbean.kten.cuda.tensor.platform

import eu.redbean.kten.api.tensor.operations.TensorOperations
import eu.redbean.kten.api.tensor.platform.DeviceType
import eu.redbean.kten.api.tensor.platform.PlatformInfo
import eu.redbean.kten.api.tensor.platform.PlatformInitializer
import eu.redbean.kten.api.tensor.platform.PlatformProvider
import eu.redbean.kten.api.tensor.store.AbstractRawTensor
import eu.redbean.kten.cuda.tensor.operations.CUDATensorOperations
import eu.redbean.kten.cuda.tensor.store.CUDARawTensor
import eu.redbean.kten.jvm.tensor.operations.JVMTensorOperations
import eu.redbean.kten.jvm.tensor.store.JVMRawTensor
import java.lang.foreign.Arena
import java.lang.foreign.ValueLayout.JAVA_INT
import java.lang.foreign.ValueLayout.JAVA_LONG

/**
 * Discovered by PlatformProvider's scan of eu.redbean.kten (PlatformProvider.kt:51-59): registers one
 * platform per CUDA device plus the JVM <-> CUDA raw-data transformers, like OCLPlatformInitializer.
 */
object CUDAPlatformInitializer : PlatformInitializer {

    override val platformKeys: List<String>

    init {
        val keys = mutableListOf<String>()
        Arena.ofConfined().use { arena ->
            val count = arena.allocate(JAVA_INT)
            KtcNative.check(KtcNative.init.invokeExact(count) as Int)          // fails without a CUDA device: there is no CPU path
            for (device in 0 until count.get(JAVA_INT, 0)) {
                val name = arena.allocate(128)
                val memory = arena.allocate(JAVA_LONG)
                val sms = arena.allocate(JAVA_INT)
                KtcNative.check(KtcNative.deviceInfo.invokeExact(device, name, 128L, memory, sms) as Int)
                val key = "CUDA - $device - ${name.getString(0)}"
                val ops = CUDATensorOperations(key, device)
                val info = PlatformInfo("CUDA", DeviceType.GPU, memory.get(JAVA_LONG, 0), key)
                @Suppress("UNCHECKED_CAST")
                PlatformProvider.register(key, ops as TensorOperations<AbstractRawTensor<Any>>, info)
                PlatformProvider.registerPlatformTransformer(JVMTensorOperations.platformKey to key) {
                    val jvm = it as JVMRawTensor
                    @Suppress("UNCHECKED_CAST")
                    ops.createRaw(jvm.shape) { i -> jvm.storeReference[i] } as AbstractRawTensor<Any>
                }
                PlatformProvider.registerPlatformTransformer(key to JVMTensorOperations.platformKey) {
                    val cuda = it as AbstractRawTensor<*> as CUDARawTensor
                    val host = cuda.toFloatArray()
                    @Suppress("UNCHECKED_CAST")
                    JVMTensorOperations.createRaw(cuda.shape) { i -> host[i] } as AbstractRawTensor<Any>
                }
                keys += key
            }
        }
        platformKeys = keys
    }
}
